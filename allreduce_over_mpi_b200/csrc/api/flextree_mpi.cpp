// MPI_Allreduce-compatible entry point (see flextree_mpi.h).
#include "flextree_mpi.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>

#include "../planner/config.hpp"
#include "../planner/cost_model.hpp"
#include "../planner/cpu_executor.hpp"

struct ft_cpu_world { ft::CpuWorld w; };  // layout shared with flextree_host.cpp

struct ft_mpi_comm {
  ft_cpu_world* threads = nullptr;  // thread world ...
  int rank = 0;
  ft_proc_world* procs = nullptr;   // ... or process world ...
  ft_comm* gpu = nullptr;           // ... or GPU communicator
  void* stream = nullptr;
  // FT_TOPO / FT_LONELY are looked up on every call like the reference does, but parsed (and the plan fetched)
  // only when their text changed since the communicator's previous call
  bool have_cfg = false;
  std::string topo_text, lonely_text;
  ft::ShapeConfig cfg;
  const ft::Plan* plan = nullptr;   // thread world: the plan of cfg.shape
};

namespace {
thread_local std::string g_err;
// The reference rebuilds its schedule on every call (mpi_mod.hpp:1520-1527); here a plan is built
// once per (world, shape) and shared by all rank threads.
const ft::Plan& plan_for(int world, const ft::Shape& shape) {
  static std::mutex mu;
  static std::map<std::string, ft::Plan> cache;
  const std::string key = std::to_string(world) + ":" + shape.str();
  std::lock_guard<std::mutex> lk(mu);
  auto it = cache.find(key);
  if (it == cache.end()) it = cache.emplace(key, ft::build_plan(world, shape)).first;
  return it->second;
}
int fail(int code, const std::string& msg) {
  g_err = msg;
  std::fprintf(stderr, "%s\n", msg.c_str());
  return code;
}
// One element of a buffer as text, for the debug dumps.
std::string value_text(int dtype, const void* base, size_t i) {
  char b[48];
  switch (dtype) {
    case FT_F32: std::snprintf(b, sizeof b, "%g", (double)((const float*)base)[i]); break;
    case FT_F64: std::snprintf(b, sizeof b, "%g", ((const double*)base)[i]); break;
    case FT_BF16: {
      unsigned u = (unsigned)((const unsigned short*)base)[i] << 16;
      float f;
      std::memcpy(&f, &u, 4);
      std::snprintf(b, sizeof b, "%g", (double)f);
      break;
    }
    case FT_F16: std::snprintf(b, sizeof b, "0x%04x", ((const unsigned short*)base)[i]); break;
    case FT_U8: case FT_BOOL: std::snprintf(b, sizeof b, "%u", ((const unsigned char*)base)[i]); break;
    case FT_I8: std::snprintf(b, sizeof b, "%d", ((const signed char*)base)[i]); break;
    case FT_U16: std::snprintf(b, sizeof b, "%u", ((const unsigned short*)base)[i]); break;
    case FT_I16: std::snprintf(b, sizeof b, "%d", ((const short*)base)[i]); break;
    case FT_I32: std::snprintf(b, sizeof b, "%d", ((const int*)base)[i]); break;
    case FT_U32: std::snprintf(b, sizeof b, "%u", ((const unsigned*)base)[i]); break;
    case FT_I64: std::snprintf(b, sizeof b, "%lld", ((const long long*)base)[i]); break;
    case FT_U64: std::snprintf(b, sizeof b, "%llu", ((const unsigned long long*)base)[i]); break;
    default: std::snprintf(b, sizeof b, "?"); break;
  }
  return b;
}
// "<label> CHECK node <rank>: v0 v1 ..." with the first 100 values of a host buffer, as one write to stderr:
// the reference's FT_DEBUG dumps after its two phases ("Med CHECK" / "Tail CHECK", mpi_mod.hpp:1601-1613, :1657-1670).
void dump_values(const char* label, int rank, int dtype, const void* host, size_t count) {
  std::string line = std::string(label) + " CHECK node " + std::to_string(rank) + ":";
  for (size_t i = 0; i < count && i < 100; ++i) line += " " + value_text(dtype, host, i);
  line += "\n";
  std::fputs(line.c_str(), stderr);
}

bool is_device_pointer(const void* p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
  return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}
}  // namespace

extern "C" {

void FT_enabled(void) { std::puts("FlexTree enabled"); }
const char* ft_mpi_last_error(void) { return g_err.c_str(); }

FT_Comm ft_mpi_thread_rank(ft_cpu_world* world, int rank) {
  if (!world || rank < 0 || rank >= world->w.n) return nullptr;
  auto* c = new ft_mpi_comm;
  c->threads = world;
  c->rank = rank;
  return c;
}
FT_Comm ft_mpi_from_comm(ft_comm* comm, void* stream) {
  if (!comm) return nullptr;
  auto* c = new ft_mpi_comm;
  c->gpu = comm;
  c->rank = ft_comm_rank(comm);
  c->stream = stream;
  return c;
}
FT_Comm ft_mpi_proc_rank(ft_proc_world* world) {
  if (!world) return nullptr;
  auto* c = new ft_mpi_comm;
  c->procs = world;
  c->rank = ft_proc_world_rank(world);
  return c;
}
FT_Comm ft_mpi_proc_init_env(double timeout_s) {
  auto env = [](const char* a, const char* b) -> const char* {
    const char* v = std::getenv(a);
    return v && *v ? v : std::getenv(b);
  };
  const char* r = env("FT_RANK", "RANK");
  const char* n = env("FT_WORLD", "WORLD_SIZE");
  const char* s = env("FT_SESSION", "MASTER_PORT");
  if (!r || !n || !s) { fail(FT_ERR_INVALID_ARG, "ft_mpi_proc_init_env: need FT_RANK/FT_WORLD/FT_SESSION (or RANK/WORLD_SIZE/MASTER_PORT)"); return nullptr; }
  char err[256];
  ft_proc_world* w = ft_proc_world_join(s, std::atoi(r), std::atoi(n), timeout_s, err, sizeof err);
  if (!w) { fail(FT_ERR_NOT_AVAILABLE, std::string("ft_mpi_proc_init_env: ") + err); return nullptr; }
  return ft_mpi_proc_rank(w);
}
void ft_mpi_proc_finalize(FT_Comm c) {
  if (!c) return;
  if (c->procs) ft_proc_world_leave(c->procs);
  delete c;
}
ft_proc_world* ft_mpi_proc_world(FT_Comm c) { return c ? c->procs : nullptr; }
int FT_Barrier(FT_Comm c) {
  if (!c) return FT_ERR_INVALID_ARG;
  if (c->procs) return ft_proc_barrier(c->procs);
  if (c->threads) {   // an all-reduce of one byte over the flat plan is a barrier
    unsigned char b = 0;
    return MPI_Allreduce_FT_c(FT_IN_PLACE, &b, 1, FT_UINT8_T, FT_OP_SUM, c);
  }
  return FT_ERR_NOT_AVAILABLE;
}
void ft_mpi_comm_free(FT_Comm c) { delete c; }

int FT_Comm_size(FT_Comm c, int* size) {
  if (!c || !size) return FT_ERR_INVALID_ARG;
  *size = c->threads ? c->threads->w.n : (c->procs ? ft_proc_world_size(c->procs) : ft_comm_world(c->gpu));
  return 0;
}
int FT_Comm_rank(FT_Comm c, int* rank) {
  if (!c || !rank) return FT_ERR_INVALID_ARG;
  *rank = c->rank;
  return 0;
}
int FT_Type_size(FT_Datatype t, int* size) {
  if (!size) return FT_ERR_INVALID_ARG;
  *size = (int)ft_dtype_size((ft_dtype)t);
  return *size ? 0 : FT_ERR_UNSUPPORTED_TYPE;
}
int FT_Type_get_name(FT_Datatype t, char* name, int* len) {
  const char* s = ft_dtype_name((ft_dtype)t);
  if (name) std::strcpy(name, s);
  if (len) *len = (int)std::strlen(s);
  return 0;
}

int MPI_Allreduce_FT_c(const void* sendbuf, void* recvbuf, size_t count, FT_Datatype datatype, FT_Op op, FT_Comm comm) {
  if (!comm || !recvbuf) return fail(FT_ERR_INVALID_ARG, "MPI_Allreduce_FT: null communicator or receive buffer");
  int world = 1;
  FT_Comm_size(comm, &world);
  const bool in_place = sendbuf == FT_IN_PLACE || sendbuf == nullptr || sendbuf == recvbuf;
  const size_t es = ft_dtype_size((ft_dtype)datatype);
  if (op != FT_SUM && op != FT_BAND) return fail(FT_ERR_UNSUPPORTED_OP, "Unsupported op " + std::to_string(op));
  if (!es || !ft_op_supported((ft_op)op, (ft_dtype)datatype))
    return fail(FT_ERR_UNSUPPORTED_TYPE, std::string("Type ") + ft_dtype_name((ft_dtype)datatype) + " is not supported in MPI mode.");

  // tree shape from the environment, on every call like the reference
  {
    const char* t = std::getenv("FT_TOPO");
    const char* l = std::getenv("FT_LONELY");
    if (!comm->have_cfg || comm->topo_text != (t ? t : "") || comm->lonely_text != (l ? l : "")) {
      comm->topo_text = t ? t : "";
      comm->lonely_text = l ? l : "";
      comm->cfg = ft::parse_topo(comm->topo_text, comm->lonely_text, world);
      comm->plan = nullptr;
      comm->have_cfg = true;
    }
  }
  const ft::ShapeConfig& cfg = comm->cfg;
  if (!cfg.ok()) return fail(FT_ERR_INVALID_TOPO, cfg.error);
  ft::Shape shape = cfg.shape;
  int debug = 0;
  if (const char* dbg = std::getenv("FT_DEBUG"); dbg && dbg[0] >= '1' && dbg[0] <= '9') debug = dbg[0] - '0';
  if (debug >= 1) {
    int rank = 0;
    FT_Comm_rank(comm, &rank);
    char line[256];
    ft_context_describe(world, rank, shape.lonely, count, datatype, line, sizeof line);
    std::fprintf(stderr, "%s", line);
  }

  // FT_DEBUG=2: the call runs as its two halves, reduce-scatter then all-gather, and every rank prints the first
  // 100 values of its buffer after each, in rank order where the world has a barrier (threads, processes).
  if (debug >= 2 && world > 1 && (comm->threads || comm->procs)) {
    if (cfg.is_auto) shape = ft::Shape::flat(world);
    if (!in_place) std::memcpy(recvbuf, sendbuf, count * es);
    const int nw = (int)shape.widths.size();
    for (int phase = 1; phase <= 2; ++phase) {
      int st3[3] = {0, 0, 0};
      const int rc = comm->threads
                         ? ft_cpu_phase(comm->threads, comm->rank, shape.widths.data(), nw, shape.lonely, shape.ring, op, datatype,
                                        recvbuf, count, 0, phase, st3)
                         : ft_proc_phase(comm->procs, shape.widths.data(), nw, shape.lonely, shape.ring, op, datatype, recvbuf, count,
                                         phase, st3);
      if (rc != FT_OK)
        return fail(rc, std::string("MPI_Allreduce_FT: ") + ft_status_name((ft_status)rc) + " at rendezvous " + std::to_string(st3[1]));
      for (int r = 0; r < world; ++r) {   // one rank at a time, the others wait (both phases end with every rank present)
        if (r == comm->rank) dump_values(phase == 1 ? "Med" : "Tail", comm->rank, datatype, recvbuf, count);
        if (comm->procs) ft_proc_barrier(comm->procs);
        else {   // an all-reduce of one byte over the flat plan is a barrier of the thread world
          unsigned char b = 0;
          ft::cpu_allreduce(comm->threads->w, comm->rank, plan_for(world, ft::Shape::flat(world)), FT_SUM, FT_U8, nullptr, &b, 1, 0,
                            nullptr, 1);
        }
      }
    }
    return 0;
  }

  if (comm->threads) {
    if (world <= 1) {
      if (!in_place) std::memcpy(recvbuf, sendbuf, count * es);
      return 0;
    }
    if (cfg.is_auto) shape = ft::Shape::flat(world);  // on shared host memory every shape moves the same bytes
    if (!comm->plan) comm->plan = &plan_for(world, shape);
    const ft::Plan& plan = *comm->plan;
    ft::RankStatus st = ft::cpu_allreduce(comm->threads->w, comm->rank, plan, (ft_op)op, (ft_dtype)datatype,
                                          in_place ? nullptr : sendbuf, recvbuf, count, 0, nullptr, 1);
    if (st.code != FT_OK)
      return fail(st.code, std::string("MPI_Allreduce_FT: ") + ft_status_name(st.code) + " at rendezvous " +
                               std::to_string(st.stage) + " (peer " + std::to_string(st.peer) + ")");
    return 0;
  }

  if (comm->procs) {
    if (cfg.is_auto) shape = ft::Shape::flat(world);
    int st3[3] = {0, 0, 0};
    const int nw = (int)shape.widths.size();
    const int rc = ft_proc_allreduce(comm->procs, shape.widths.data(), nw, shape.lonely, shape.ring, op, datatype,
                                     in_place ? nullptr : sendbuf, recvbuf, count, st3);
    if (rc != FT_OK)
      return fail(rc, std::string("MPI_Allreduce_FT: ") + ft_status_name((ft_status)rc) + " at rendezvous " + std::to_string(st3[1]) +
                          " (peer " + std::to_string(st3[2]) + ") " + ft_proc_last_error(comm->procs));
    return 0;
  }

  // ---- GPU communicator
  ft_comm* g = comm->gpu;
  const int nw = cfg.is_auto ? 0 : (int)shape.widths.size();
  const int* widths = cfg.is_auto ? nullptr : shape.widths.data();
  const int explicit_shape = !(cfg.is_auto || (!std::getenv("FT_TOPO") && !std::getenv("FT_LONELY")));
  // AUTO either way: with a shape from the environment that plan runs (on tagged words while the message is small, through
  // the staged kernel above that); without one the selection policy picks algorithm and shape
  const int algo = FT_ALGO_AUTO;
  const bool dev_recv = is_device_pointer(recvbuf);
  const bool dev_send = in_place ? dev_recv : is_device_pointer(sendbuf);
  if (debug >= 2 && world > 1 && dev_recv && dev_send) {
    // GPU ranks: the halves as collectives of their own on a heap tensor, a host copy of the first 100 values after
    // each; ranks are separate processes without a barrier of their own here, so every dump is one prefixed line
    const ft::Shape sh = explicit_shape ? shape : ft::Shape::flat(world);
    cudaStream_t st = (cudaStream_t)comm->stream;
    if (!in_place && cudaMemcpyAsync(recvbuf, sendbuf, count * es, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
      return fail(FT_ERR_CUDA, "MPI_Allreduce_FT: device copy failed");
    unsigned char head[100 * 8];
    const size_t n = count < 100 ? count : 100;
    for (int phase = 1; phase <= 2; ++phase) {
      int rc = phase == 1 ? ft_reduce_scatter(g, recvbuf, count, datatype, op, sh.widths.data(), (int)sh.widths.size(), sh.lonely, sh.ring, 1.0f, comm->stream)
                          : ft_all_gather(g, recvbuf, count, datatype, sh.widths.data(), (int)sh.widths.size(), sh.lonely, sh.ring, comm->stream);
      if (rc != FT_OK) return fail(rc, ft_comm_last_error(g));
      if (cudaMemcpyAsync(head, recvbuf, n * es, cudaMemcpyDeviceToHost, st) != cudaSuccess || cudaStreamSynchronize(st) != cudaSuccess)
        return fail(FT_ERR_CUDA, "MPI_Allreduce_FT: debug copy failed");
      dump_values(phase == 1 ? "Med" : "Tail", comm->rank, datatype, head, n);
    }
    return 0;
  }
  if (dev_recv && dev_send) {
    int rc = ft_allreduce(g, in_place ? nullptr : sendbuf, recvbuf, count, datatype, op, explicit_shape ? widths : nullptr,
                          explicit_shape ? nw : 0, explicit_shape ? shape.lonely : 0, explicit_shape ? shape.ring : 0, algo,
                          1.0f, comm->stream);
    if (rc != FT_OK) return fail(rc, ft_comm_last_error(g));
    return 0;
  }
  // Host buffers (the reference's only kind): pipelined through the GPU, see ft_allreduce_host.  A call that mixes
  // a host and a device buffer is first brought to one side with a plain copy.
  cudaStream_t st = (cudaStream_t)comm->stream;
  const size_t bytes = count * es;
  if (dev_recv) {   // host source, device result
    if (cudaMemcpyAsync(recvbuf, sendbuf, bytes, cudaMemcpyHostToDevice, st) != cudaSuccess)
      return fail(FT_ERR_CUDA, "MPI_Allreduce_FT: host-to-device copy failed");
    int rc = ft_allreduce(g, nullptr, recvbuf, count, datatype, op, explicit_shape ? widths : nullptr, explicit_shape ? nw : 0,
                          explicit_shape ? shape.lonely : 0, explicit_shape ? shape.ring : 0, algo, 1.0f, comm->stream);
    if (rc != FT_OK) return fail(rc, ft_comm_last_error(g));
    return 0;
  }
  if (dev_send && !in_place) {   // device source, host result
    if (cudaMemcpyAsync(recvbuf, sendbuf, bytes, cudaMemcpyDeviceToHost, st) != cudaSuccess || cudaStreamSynchronize(st) != cudaSuccess)
      return fail(FT_ERR_CUDA, "MPI_Allreduce_FT: device-to-host copy failed");
    sendbuf = nullptr;
  }
  {
    int rc = ft_allreduce_host(g, in_place || !sendbuf ? nullptr : sendbuf, recvbuf, count, datatype, op,
                               explicit_shape ? widths : nullptr, explicit_shape ? nw : 0, explicit_shape ? shape.lonely : 0,
                               explicit_shape ? shape.ring : 0, algo, 1.0f, comm->stream);
    if (rc != FT_OK) return fail(rc, ft_comm_last_error(g));
    if (cudaStreamSynchronize(st) != cudaSuccess) return fail(FT_ERR_CUDA, "MPI_Allreduce_FT: the pipelined host all-reduce failed");
  }
  int status[5];
  if (ft_comm_status(g, status) != FT_OK)
    return fail(status[0], std::string("MPI_Allreduce_FT: ") + ft_status_name((ft_status)status[0]) + " waiting for rank " + std::to_string(status[2]));
  return 0;
}

int MPI_Allreduce_FT(const void* sendbuf, void* recvbuf, int count, FT_Datatype datatype, FT_Op op, FT_Comm comm) {
  if (count < 0) return fail(FT_ERR_INVALID_ARG, "MPI_Allreduce_FT: negative count");
  return MPI_Allreduce_FT_c(sendbuf, recvbuf, (size_t)count, datatype, op, comm);
}

}  // extern "C"
