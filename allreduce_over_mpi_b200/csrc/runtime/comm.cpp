// FlexTree communicator runtime: symmetric heaps, peer mappings, NVLS multicast binding,
// device plan tables and the host side of every collective launch.
//
// The CUDA driver API (virtual memory management, multicast objects) is resolved at run
// time through cudaGetDriverEntryPoint, so the library has no link-time dependency on
// libcuda and still loads on a machine without a driver.
//
// Reference counterpart: FlexTree_Context (allreduce_over_mpi/mpi_mod.hpp:776-809), the
// grow-only staging buffer (:1489-1507), the entry point's dispatch (:1723-1778) and
// tree_allreduce's per-call planning (:1520-1548) — with the plan cached per shape
// instead of rebuilt on every call.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../api/flextree.h"
#include "../api/flextree_comm.h"
#include "../api/policy_handle.hpp"
#include "../kernels/comm_bounds.h"
#include "../kernels/comm_dev.h"
#include "../kernels/pol_ids.h"
#include "../planner/plan.hpp"
#include "dev_plan.hpp"
#include "heap_alloc.hpp"
#include <unistd.h>

namespace ftk {
cudaError_t launch_staged(int pol, const CommDev& c, const StagedArgs& a, int lanes, cudaStream_t st);
cudaError_t launch_oneshot(int pol, const CommDev& c, const OneShotArgs& a, uint64_t slot_bytes, int lanes, cudaStream_t st);
cudaError_t launch_nvls(int pol, const CommDev& c, const NvlsArgs& a, int lanes, int mode, const NvlsConfig& cfg, cudaStream_t st);
cudaError_t launch_push(int pol, const CommDev& c, const NvlsArgs& a, int lanes, bool do_sync, cudaStream_t st);
cudaError_t launch_ll(int pol, const CommDev& c, const LLArgs& a, cudaStream_t st);
cudaError_t launch_hybrid(int pol, const CommDev& c, const NvlsArgs& a, int lanes, int nvls_lanes, uint64_t nvls_bytes, cudaStream_t st);
cudaError_t launch_ll_tree(int pol, const CommDev& c, const LLTreeArgs& a, cudaStream_t st);
cudaError_t launch_nvls_oneshot(int pol, const CommDev& c, const OneShotArgs& a, uint64_t slot_bytes, int lanes, int threads, cudaStream_t st);
cudaError_t launch_wait_probe(const CommDev& c, int peer, unsigned long long timeout_ns, cudaStream_t st);
}  // namespace ftk

namespace {

// ---- driver API, resolved lazily -------------------------------------------------------
struct Driver {
  bool ok = false;
  std::string why;
#define FT_DRV(name) decltype(&name) p_##name = nullptr;
  FT_DRV(cuMemCreate) FT_DRV(cuMemRelease) FT_DRV(cuMemGetAllocationGranularity) FT_DRV(cuMemAddressReserve)
  FT_DRV(cuMemAddressFree) FT_DRV(cuMemMap) FT_DRV(cuMemUnmap) FT_DRV(cuMemSetAccess)
  FT_DRV(cuMemExportToShareableHandle) FT_DRV(cuMemImportFromShareableHandle) FT_DRV(cuDeviceGetAttribute)
  FT_DRV(cuMulticastCreate) FT_DRV(cuMulticastAddDevice) FT_DRV(cuMulticastBindMem) FT_DRV(cuMulticastUnbind)
  FT_DRV(cuMulticastGetGranularity) FT_DRV(cuGetErrorString)
#undef FT_DRV
};

Driver& driver() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    cudaFree(nullptr);  // make sure the runtime (and with it the driver) is initialised
    auto get = [&](const char* name, void** fn) {
      cudaDriverEntryPointQueryResult q;
      if (cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !*fn) {
        if (d.why.empty()) d.why = std::string("driver entry point missing: ") + name;
        cudaGetLastError();
        return false;
      }
      return true;
    };
    bool all = true;
#define FT_GET(name) all = get(#name, (void**)&d.p_##name) && all;
    FT_GET(cuMemCreate) FT_GET(cuMemRelease) FT_GET(cuMemGetAllocationGranularity) FT_GET(cuMemAddressReserve)
    FT_GET(cuMemAddressFree) FT_GET(cuMemMap) FT_GET(cuMemUnmap) FT_GET(cuMemSetAccess)
    FT_GET(cuMemExportToShareableHandle) FT_GET(cuMemImportFromShareableHandle) FT_GET(cuDeviceGetAttribute)
    FT_GET(cuGetErrorString)
#undef FT_GET
    d.ok = all;
    // multicast is optional
    get("cuMulticastCreate", (void**)&d.p_cuMulticastCreate);
    get("cuMulticastAddDevice", (void**)&d.p_cuMulticastAddDevice);
    get("cuMulticastBindMem", (void**)&d.p_cuMulticastBindMem);
    get("cuMulticastUnbind", (void**)&d.p_cuMulticastUnbind);
    get("cuMulticastGetGranularity", (void**)&d.p_cuMulticastGetGranularity);
  });
  return d;
}

std::string cu_err(CUresult r) {
  const char* s = nullptr;
  if (driver().p_cuGetErrorString) driver().p_cuGetErrorString(r, &s);
  return s ? s : ("CUresult " + std::to_string((int)r));
}

constexpr size_t kFlagBytes = (size_t)ftk::kMaxLanes * FT_MAX_RANKS * sizeof(ftk::flag_t);
size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// The multicast object of a world.  Ranks that live in one process share ONE driver handle, which must
// outlive every rank's binding and mapping: the last rank to let go releases it.
struct McOwner {
  CUmemGenericAllocationHandle h = 0;
  explicit McOwner(CUmemGenericAllocationHandle handle) : h(handle) {}
  ~McOwner() { if (h && driver().p_cuMemRelease) driver().p_cuMemRelease(h); }
};

struct DevPlanEntry {
  ftk::DevPlan* plan = nullptr;   // device
  ftk::DevPull* pulls = nullptr;  // device
  ftk::DevPush* pushes = nullptr; // device: the plan's edges seen from their source (tagged-word form)
  int nstages = 0;
  uint32_t nslots = 0;            // receive slots this rank needs in the tagged-word form
  uint32_t npulls = 0, npushes = 0;
};

}  // namespace

struct ft_comm {
  int rank = 0, world = 1, device = 0, mem_kind = FT_MEM_VMM;
  size_t user_bytes = 0, staging_bytes = 0, total_bytes = 0, staging_off = 0, ll_off = 0, flags_off = 0;
  ft::HeapAllocator heap_alloc;   // offsets of the tensors handed out from the user part of the heap
  // host-side usage counters per algorithm (FT_ALGO_* index; 7 = reduce-scatter alone, 8 = all-gather alone, 9 = FT_ALGO_NVLS1)
  uint64_t stat_calls[10] = {}, stat_bytes[10] = {};
  // local allocation
  CUmemGenericAllocationHandle handle = 0;
  CUdeviceptr va = 0;
  void* ipc_ptr = nullptr;
  // peers
  unsigned char* peer_base[FT_MAX_RANKS] = {};
  CUmemGenericAllocationHandle peer_handle[FT_MAX_RANKS] = {};
  bool peer_is_ipc[FT_MAX_RANKS] = {};
  bool peer_is_vmm[FT_MAX_RANKS] = {};
  // multicast
  CUmemGenericAllocationHandle mc_handle = 0;
  std::shared_ptr<McOwner> mc_owner;   // releases mc_handle when the last holder is gone
  CUdeviceptr mc_va = 0;
  bool mc_have = false, mc_joined = false, mc_bound = false;
  // local device state
  unsigned long long* call_count = nullptr;
  unsigned int* arrived = nullptr;
  ftk::Status* status_host = nullptr;
  ftk::Status* status_dev = nullptr;
  double timeout_ms = 10000.0;
  int max_lanes = 0, sms = 148;
  size_t oneshot_max = 64 << 10;
  double hybrid_fraction = 0.7, hybrid_lane_fraction = 0.5;
  size_t ll_max = 8 << 10;   // AUTO uses the low-latency protocol up to this size
  int nvls_ctas_per_sm = 1;   // measured on 8 GPUs: 2 or 3 CTAs per SM lose 5-15 % at 256 MiB and above
  ftk::NvlsConfig nvls_cfg;   // threads per CTA, vectors in flight per thread, instruction form
  int nvls_max_lanes = 32;    // 0: as many lanes as SMs (times nvls_ctas_per_sm).  8 GPUs, 64 MiB / 256 MiB / 1 GiB: 32 CTAs of
                              // 256 threads reach 683 / 806 / 839 GB/s, all 148 SMs 632 / 786 / 834, 16 CTAs 682 / 797 / 828
  size_t nvls_stripe = 0;
  int nvls1_max_lanes = 64;   // CTAs of the one-shot-through-the-switch kernel (0: one per SM)
  int phase_nvls = 1;         // ft_reduce_scatter / ft_all_gather through the multimem kernels (flat shape, eligible tensor):
                              // 0 never, 1 where it measured faster (five ranks and more), 2 whenever possible     // all-reduce: 0 = rank r owns block r, else round-robin stripes of this many bytes
  std::map<std::string, DevPlanEntry> plans;
  // ft_allreduce_host: chunk buffers in the heap + three streams, made on first use
  struct HostPipe {
    static constexpr int kDepth = 3;
    cudaStream_t in = nullptr, run = nullptr, out = nullptr;
    cudaEvent_t start = nullptr, in_done[kDepth] = {}, run_done[kDepth] = {}, out_done[kDepth] = {};
    unsigned char* slot[kDepth] = {};
    size_t chunk = 0;
    bool used[kDepth] = {};
  } hp;
  size_t host_chunk_bytes = 32u << 20;
  size_t ll_tree_max = 64u << 10;   // AUTO with an explicit shape: tagged-word form of the plan up to this size
  int forced_algo = FT_ALGO_AUTO;   // FT_ALGO=<name> in the environment: what AUTO resolves to, whatever the size
  ft_policy* policy = nullptr;   // algorithm / shape per message size (calibration table + cost model)
  ftk::CommDev dev{};
  bool finalized = false;
  std::string err;
};

namespace {

int fail(ft_comm* c, int code, const std::string& what) {
  if (c) c->err = what;
  return code;
}
#define FT_CUDA(c, call)                                                                        \
  do {                                                                                          \
    cudaError_t e_ = (call);                                                                    \
    if (e_ != cudaSuccess) return fail(c, FT_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_)); \
  } while (0)
#define FT_CU(c, call)                                                                          \
  do {                                                                                          \
    CUresult r_ = (call);                                                                       \
    if (r_ != CUDA_SUCCESS) return fail(c, FT_ERR_CUDA, std::string(#call) + ": " + cu_err(r_)); \
  } while (0)

CUmemAllocationProp vmm_prop(int device) {
  CUmemAllocationProp p{};
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

int map_handle(ft_comm* c, CUmemGenericAllocationHandle h, size_t bytes, CUdeviceptr* out) {
  Driver& d = driver();
  CUdeviceptr va = 0;
  FT_CU(c, d.p_cuMemAddressReserve(&va, bytes, 0, 0, 0));
  FT_CU(c, d.p_cuMemMap(va, bytes, 0, h, 0));
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = c->device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  FT_CU(c, d.p_cuMemSetAccess(va, bytes, &acc, 1));
  *out = va;
  return FT_OK;
}

unsigned char* local_base(ft_comm* c) { return c->mem_kind == FT_MEM_VMM ? (unsigned char*)c->va : (unsigned char*)c->ipc_ptr; }

ft::Shape make_shape(int world, const int* widths, int nw, int lonely, int ring) {
  ft::Shape s;
  if (widths && nw > 0) s.widths.assign(widths, widths + nw);
  else s.widths = {world};
  s.lonely = lonely;
  s.ring = ring != 0;
  return s;
}

// Build (once per shape) this rank's device plan table.
int get_plan(ft_comm* c, const ft::Shape& shape, DevPlanEntry** out) {
  const std::string key = shape.str();
  auto it = c->plans.find(key);
  if (it != c->plans.end()) { *out = &it->second; return FT_OK; }
  ft::Plan p = ft::build_plan(c->world, shape);
  if (!p.ok()) return fail(c, FT_ERR_INVALID_TOPO, "invalid FT_TOPO " + key + " (" + p.error + ")");
  if (p.num_stages > ftk::kMaxStages) return fail(c, FT_ERR_TOO_LARGE, "plan has too many stages");
  ft::HostDevPlan hd = ft::build_dev_plan(p, c->rank);
  const std::string flaw = ft::check_dev_plan(hd, c->world, c->rank);
  if (!flaw.empty()) return fail(c, FT_ERR_INVALID_TOPO, "plan " + key + " failed its descriptor check (" + flaw + ")");
  const ftk::DevPlan& hp = hd.plan;
  const std::vector<ftk::DevPull>& pulls = hd.pulls;
  DevPlanEntry e;
  e.nstages = p.num_stages;
  FT_CUDA(c, cudaMalloc(&e.plan, sizeof(ftk::DevPlan)));
  FT_CUDA(c, cudaMalloc(&e.pulls, sizeof(ftk::DevPull) * (pulls.size() + 1)));
  FT_CUDA(c, cudaMemcpy(e.plan, &hp, sizeof hp, cudaMemcpyHostToDevice));
  if (!pulls.empty()) FT_CUDA(c, cudaMemcpy(e.pulls, pulls.data(), sizeof(ftk::DevPull) * pulls.size(), cudaMemcpyHostToDevice));
  FT_CUDA(c, cudaMalloc(&e.pushes, sizeof(ftk::DevPush) * (hd.pushes.size() + 1)));
  if (!hd.pushes.empty())
    FT_CUDA(c, cudaMemcpy(e.pushes, hd.pushes.data(), sizeof(ftk::DevPush) * hd.pushes.size(), cudaMemcpyHostToDevice));
  e.nslots = hp.nslots;
  e.npulls = (uint32_t)pulls.size();
  e.npushes = (uint32_t)hd.pushes.size();
  *out = &c->plans.emplace(key, e).first->second;
  return FT_OK;
}

// In the heap AND on a 16-byte boundary: only then may the kernels address the tensor in place with
// vector loads.  A slice of a heap tensor that starts at an odd element is treated like any other
// user tensor (staged through the slots, where alignment is handled element by element).
bool in_heap(ft_comm* c, const void* p, size_t bytes) {
  const unsigned char* b = local_base(c);
  const unsigned char* q = (const unsigned char*)p;
  return b && q >= b && q + bytes <= b + c->user_bytes && ((uintptr_t)q & 15) == 0;
}

// Elements per block: ceil(count/world) rounded up so that a block is a whole number of 16-byte vectors
// (trailing blocks come out short or empty, like the reference's split); blocks of 64 KiB and more are whole
// multiples of 512 bytes, so that every block (and with it every lane's slice) starts on a warp-request boundary.
uint64_t pick_block_elems(uint64_t count, int world, uint32_t es) {
  uint64_t b = (count + world - 1) / (uint64_t)world;
  const uint64_t per = (b * es >= (64u << 10) ? 512 : 16) / es;
  b = (b + per - 1) / per * per;
  return b ? b : 16 / es;
}

int pick_lanes(ft_comm* c, uint64_t region_bytes, uint64_t min_chunk, int ctas_per_sm = 1) {
  uint64_t lanes = region_bytes / min_chunk;
  if (lanes < 1) lanes = 1;
  const int cap = c->max_lanes > 0 ? c->max_lanes : c->sms * ctas_per_sm;
  if (lanes > (uint64_t)cap) lanes = cap;
  if (lanes > (uint64_t)ftk::kMaxLanes) lanes = ftk::kMaxLanes;
  return (int)lanes;
}

struct Prepared {
  int pol;
  uint32_t es;
  uint64_t bytes;
  bool heap_resident;
};
int prepare(ft_comm* c, const void* sendbuf, void* recvbuf, size_t count, int dtype, int op, Prepared* out) {
  if (!c || !c->finalized) return fail(c, FT_ERR_INVALID_ARG, "communicator not finalized");
  if (op < 0 || op >= FT_OP_COUNT) return fail(c, FT_ERR_UNSUPPORTED_OP, "Unsupported op " + std::to_string(op));
  const int pol = ftk::policy_id(op, dtype);
  if (pol < 0) return fail(c, FT_ERR_UNSUPPORTED_TYPE, std::string("Type ") + ft_dtype_name((ft_dtype)dtype) + " is not supported");
  if (!recvbuf && count) return fail(c, FT_ERR_INVALID_ARG, "recvbuf is null");
  out->pol = pol;
  out->es = (uint32_t)ft_dtype_size((ft_dtype)dtype);
  out->bytes = (uint64_t)count * out->es;
  out->heap_resident = in_heap(c, recvbuf, out->bytes);
  (void)sendbuf;
  return FT_OK;
}

bool nvls_eligible(ft_comm* c, const Prepared& pr) {
  return c->mc_bound && c->mc_va && pr.heap_resident && pr.bytes % 16 == 0 &&
         (pr.pol == ftk::POL_F32 || pr.pol == ftk::POL_BF16 || pr.pol == ftk::POL_F16);
}
ft::PolicyChoice choose_for(ft_comm* c, const Prepared& pr) {
  if (!c->policy) {   // a communicator that was never finalized still answers from the model
    c->policy = new ft_policy(c->world);
  }
  const bool nvls1_ok = c->mc_bound && c->mc_va && (pr.pol == ftk::POL_F32 || pr.pol == ftk::POL_BF16 || pr.pol == ftk::POL_F16);
  return c->policy->p.choose(pr.bytes, pr.heap_resident, nvls_eligible(c, pr), c->staging_bytes, c->ll_max, nvls1_ok);
}

int launch_staged_call(ft_comm* c, const Prepared& pr, const void* sendbuf, void* recvbuf, size_t count,
                       const ft::Shape& shape, float scale, int stage_begin, int stage_end, bool do_sync, cudaStream_t st,
                       bool phase_alone = false) {
  DevPlanEntry* pe = nullptr;
  int rc = get_plan(c, shape, &pe);
  if (rc != FT_OK) return rc;
  ftk::StagedArgs a{};
  a.plan = pe->plan;
  a.pulls = pe->pulls;
  a.count = count;
  a.elem_size = pr.es;
  a.block_elems = pick_block_elems(count, c->world, pr.es);
  a.scale = scale;
  a.do_sync = do_sync ? 1 : 0;
  a.stage_begin = stage_begin < 0 ? 0 : (uint32_t)stage_begin;
  a.stage_end = stage_end < 0 ? (uint32_t)pe->nstages : (uint32_t)stage_end;
  if (pr.heap_resident) {
    if (sendbuf && sendbuf != recvbuf) {
      if (a.stage_begin == 0) FT_CUDA(c, cudaMemcpyAsync(recvbuf, sendbuf, pr.bytes, cudaMemcpyDeviceToDevice, st));
    }
    a.work_off = (uint64_t)((unsigned char*)recvbuf - local_base(c));
    a.alt_stride = 0;
    a.end_sync = phase_alone ? 2 : 1;
    a.user_vec_ok = 1;
  } else {
    if (phase_alone) return fail(c, FT_ERR_INVALID_ARG, "reduce-scatter / all-gather work in place on a tensor in the symmetric heap");
    if (pr.bytes > c->staging_bytes)
      return fail(c, FT_ERR_TOO_LARGE, "message of " + std::to_string(pr.bytes) + " bytes exceeds the staging slot (" +
                                           std::to_string(c->staging_bytes) + "); allocate the tensor in the symmetric heap or split it");
    a.work_off = c->staging_off;
    a.alt_stride = c->staging_bytes;
    a.user_in = sendbuf ? sendbuf : recvbuf;
    a.user_out = recvbuf;
    a.end_sync = 0;
    a.user_vec_ok = (((uintptr_t)a.user_in | (uintptr_t)a.user_out) & 15) == 0;
  }
  const int lanes = pick_lanes(c, a.block_elems * pr.es, 8192);
  cudaError_t e = ftk::launch_staged(pr.pol, c->dev, a, lanes, st);
  if (e != cudaSuccess) return fail(c, FT_ERR_CUDA, std::string("staged launch: ") + cudaGetErrorString(e));
  return FT_OK;
}

int launch_oneshot_call(ft_comm* c, const Prepared& pr, const void* sendbuf, void* recvbuf, size_t count, float scale,
                        uint32_t phase_mask, uint64_t emu_call, cudaStream_t st) {
  if (pr.bytes > c->staging_bytes) return fail(c, FT_ERR_TOO_LARGE, "one-shot message exceeds the staging slot");
  ftk::OneShotArgs a{};
  a.slot_off = c->staging_off;
  a.emu_call = emu_call;
  a.user_in = sendbuf ? sendbuf : recvbuf;
  a.user_out = recvbuf;
  a.count = count;
  a.elem_size = pr.es;
  a.phase_mask = phase_mask;
  a.user_vec_ok = (((uintptr_t)a.user_in | (uintptr_t)a.user_out) & 15) == 0;
  a.scale = scale;
  const int lanes = pick_lanes(c, pr.bytes, 4096);
  cudaError_t e = ftk::launch_oneshot(pr.pol, c->dev, a, c->staging_bytes, lanes, st);
  if (e != cudaSuccess) return fail(c, FT_ERR_CUDA, std::string("one-shot launch: ") + cudaGetErrorString(e));
  return FT_OK;
}

int launch_push_call(ft_comm* c, const Prepared& pr, const void* sendbuf, void* recvbuf, size_t count, float scale, bool do_sync,
                     cudaStream_t st) {
  if (!pr.heap_resident) return fail(c, FT_ERR_INVALID_ARG, "the reduce+push all-reduce needs a 16-byte aligned tensor in the symmetric heap");
  if (sendbuf && sendbuf != recvbuf) FT_CUDA(c, cudaMemcpyAsync(recvbuf, sendbuf, pr.bytes, cudaMemcpyDeviceToDevice, st));
  ftk::NvlsArgs a{};
  a.work_off = (uint64_t)((unsigned char*)recvbuf - local_base(c));
  a.count = count;
  a.elem_size = pr.es;
  a.block_elems = pick_block_elems(count, c->world, pr.es);
  a.scale = scale;
  const int lanes = pick_lanes(c, a.block_elems * pr.es, 8192);
  cudaError_t e = ftk::launch_push(pr.pol, c->dev, a, lanes, do_sync, st);
  if (e != cudaSuccess) return fail(c, FT_ERR_CUDA, std::string("push launch: ") + cudaGetErrorString(e));
  return FT_OK;
}

// A plan with the tagged-word protocol.  Fits when the message is at most kLLMaxBytes and this rank's receive slots
// (two wire bytes per payload byte, one block each) fit one parity of the low-latency area.
bool ll_tree_fits(ft_comm* c, const Prepared& pr, size_t count, uint32_t nslots) {
  const uint64_t block_bytes = pick_block_elems(count, c->world, pr.es) * pr.es;
  return pr.bytes <= ftk::kLLMaxBytes && (uint64_t)nslots * 2 * block_bytes <= (uint64_t)c->world * ftk::kLLSrcStride;
}
int launch_ll_tree_call(ft_comm* c, const Prepared& pr, const void* sendbuf, void* recvbuf, size_t count, const ft::Shape& shape,
                        float scale, int stage_begin, int stage_end, uint32_t phase_mask, bool use_counter, uint64_t emu_call,
                        cudaStream_t st) {
  DevPlanEntry* pe = nullptr;
  int rc = get_plan(c, shape, &pe);
  if (rc != FT_OK) return rc;
  if (!ll_tree_fits(c, pr, count, pe->nslots))
    return fail(c, FT_ERR_TOO_LARGE, "message too large for the tagged-word form of plan " + shape.str());
  ftk::LLTreeArgs a{};
  a.plan = pe->plan;
  a.pulls = pe->pulls;
  a.pushes = pe->pushes;
  a.ll_off = c->ll_off;
  a.user_in = sendbuf ? sendbuf : recvbuf;
  a.user_out = recvbuf;
  a.count = count;
  a.block_elems = pick_block_elems(count, c->world, pr.es);
  a.elem_size = pr.es;
  a.stage_begin = stage_begin < 0 ? 0 : (uint32_t)stage_begin;
  a.stage_end = stage_end < 0 ? (uint32_t)pe->nstages : (uint32_t)stage_end;
  a.phase_mask = phase_mask;
  a.user_vec_ok = (((uintptr_t)a.user_in | (uintptr_t)a.user_out) & 15) == 0;
  a.use_call_counter = use_counter ? 1 : 0;
  a.emu_call = emu_call;
  a.scale = scale;
  const size_t tables = (size_t)pe->nstages * sizeof(ftk::DevStage) + (size_t)pe->npulls * sizeof(ftk::DevPull) +
                        (size_t)pe->npushes * sizeof(ftk::DevPush);
  if (tables <= 40 * 1024) {   // below the 48 KiB a kernel may use without opting in
    a.table_bytes = (uint32_t)((tables + 15) / 16 * 16);
    a.table_counts[0] = (uint32_t)pe->nstages;
    a.table_counts[1] = pe->npulls;
    a.table_counts[2] = pe->npushes;
  }
  cudaError_t e = ftk::launch_ll_tree(pr.pol, c->dev, a, st);
  if (e != cudaSuccess) return fail(c, FT_ERR_CUDA, std::string("tagged-word plan launch: ") + cudaGetErrorString(e));
  return FT_OK;
}

int launch_ll_call(ft_comm* c, const Prepared& pr, const void* sendbuf, void* recvbuf, size_t count, float scale,
                   uint32_t phase_mask, bool use_counter, uint64_t emu_call, cudaStream_t st) {
  if (pr.bytes > ftk::kLLMaxBytes) return fail(c, FT_ERR_TOO_LARGE, "low-latency all-reduce is limited to 256 KiB");
  ftk::LLArgs a{};
  a.ll_off = c->ll_off;
  a.user_in = sendbuf ? sendbuf : recvbuf;
  a.user_out = recvbuf;
  a.count = count;
  a.elem_size = pr.es;
  a.phase_mask = phase_mask;
  a.user_vec_ok = (((uintptr_t)a.user_in | (uintptr_t)a.user_out) & 15) == 0;
  a.use_call_counter = use_counter ? 1 : 0;
  a.emu_call = emu_call;
  a.scale = scale;
  cudaError_t e = ftk::launch_ll(pr.pol, c->dev, a, st);
  if (e != cudaSuccess) return fail(c, FT_ERR_CUDA, std::string("low-latency launch: ") + cudaGetErrorString(e));
  return FT_OK;
}

}  // namespace

extern "C" {

int ft_comm_create(int rank, int world, int device, size_t heap_bytes, size_t staging_bytes, int mem_kind, ft_comm** out) {
  if (!out || world < 1 || world > FT_MAX_RANKS || rank < 0 || rank >= world) return FT_ERR_INVALID_ARG;
  ft_comm* c = new ft_comm;
  *out = c;
  c->rank = rank; c->world = world; c->device = device; c->mem_kind = mem_kind;
  FT_CUDA(c, cudaSetDevice(device));
  FT_CUDA(c, cudaFree(nullptr));
  cudaDeviceGetAttribute(&c->sms, cudaDevAttrMultiProcessorCount, device);
  c->user_bytes = round_up(heap_bytes, 256);
  c->heap_alloc.reset(c->user_bytes);
  c->staging_bytes = round_up(staging_bytes ? staging_bytes : 256, 256);
  c->staging_off = c->user_bytes;
  c->ll_off = round_up(c->staging_off + 2 * c->staging_bytes, 4096);
  const size_t ll_bytes = 2 * (size_t)world * ftk::kLLSrcStride;   // two parities of the low-latency receive area
  c->flags_off = round_up(c->ll_off + ll_bytes, 4096);
  size_t total = c->flags_off + kFlagBytes;
  if (mem_kind == FT_MEM_VMM) {
    Driver& d = driver();
    if (!d.ok) return fail(c, FT_ERR_NOT_AVAILABLE, "CUDA VMM driver API unavailable: " + d.why);
    CUmemAllocationProp prop = vmm_prop(device);
    size_t gran = 0;
    FT_CU(c, d.p_cuMemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
    int mc = 0;
    d.p_cuDeviceGetAttribute(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device);
    if (mc && d.p_cuMulticastGetGranularity) {
      CUmulticastObjectProp mp{};
      mp.numDevices = (unsigned)world;
      mp.size = round_up(total, gran);
      mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
      size_t mg = 0;
      if (d.p_cuMulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > gran) gran = mg;
    }
    total = round_up(total, gran);
    FT_CU(c, d.p_cuMemCreate(&c->handle, total, &prop, 0));
    c->total_bytes = total;
    int rc = map_handle(c, c->handle, total, &c->va);
    if (rc != FT_OK) return rc;
  } else {
    total = round_up(total, 2 << 20);
    FT_CUDA(c, cudaMalloc(&c->ipc_ptr, total));
    c->total_bytes = total;
  }
  FT_CUDA(c, cudaMemset(local_base(c) + c->ll_off, 0, c->flags_off - c->ll_off + kFlagBytes));
  FT_CUDA(c, cudaMalloc(&c->call_count, sizeof(unsigned long long)));
  FT_CUDA(c, cudaMalloc(&c->arrived, sizeof(unsigned int)));
  FT_CUDA(c, cudaMemset(c->call_count, 0, sizeof(unsigned long long)));
  FT_CUDA(c, cudaMemset(c->arrived, 0, sizeof(unsigned int)));
  FT_CUDA(c, cudaHostAlloc(&c->status_host, sizeof(ftk::Status), cudaHostAllocMapped));
  std::memset(c->status_host, 0, sizeof(ftk::Status));
  FT_CUDA(c, cudaHostGetDevicePointer((void**)&c->status_dev, c->status_host, 0));
  c->peer_base[rank] = local_base(c);
  FT_CUDA(c, cudaDeviceSynchronize());
  return FT_OK;
}

int ft_comm_destroy(ft_comm* c) {
  if (!c) return FT_OK;
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();
  Driver& d = driver();
  if (d.ok && (c->mc_bound || c->mc_joined || c->mc_have)) {
    if (c->mc_va) { d.p_cuMemUnmap(c->mc_va, c->total_bytes); d.p_cuMemAddressFree(c->mc_va, c->total_bytes); }
    if (c->mc_bound && d.p_cuMulticastUnbind) d.p_cuMulticastUnbind(c->mc_handle, c->device, 0, c->total_bytes);
    c->mc_owner.reset();   // the handle is released with its last holder
  }
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank || !c->peer_base[r]) continue;
    if (c->peer_is_vmm[r] && d.ok) {
      d.p_cuMemUnmap((CUdeviceptr)c->peer_base[r], c->total_bytes);
      d.p_cuMemAddressFree((CUdeviceptr)c->peer_base[r], c->total_bytes);
      d.p_cuMemRelease(c->peer_handle[r]);
    } else if (c->peer_is_ipc[r]) {
      cudaIpcCloseMemHandle(c->peer_base[r]);
    }
  }
  if (c->mem_kind == FT_MEM_VMM && c->va && d.ok) {
    d.p_cuMemUnmap(c->va, c->total_bytes);
    d.p_cuMemAddressFree(c->va, c->total_bytes);
    d.p_cuMemRelease(c->handle);
  } else if (c->ipc_ptr) {
    cudaFree(c->ipc_ptr);
  }
  for (auto& kv : c->plans) { cudaFree(kv.second.plan); cudaFree(kv.second.pulls); cudaFree(kv.second.pushes); }
  if (c->hp.in) {
    cudaStreamDestroy(c->hp.in); cudaStreamDestroy(c->hp.run); cudaStreamDestroy(c->hp.out);
    cudaEventDestroy(c->hp.start);
    for (int k = 0; k < ft_comm::HostPipe::kDepth; ++k) {
      cudaEventDestroy(c->hp.in_done[k]); cudaEventDestroy(c->hp.run_done[k]); cudaEventDestroy(c->hp.out_done[k]);
    }
  }
  delete c->policy;
  cudaFree(c->call_count);
  cudaFree(c->arrived);
  if (c->status_host) cudaFreeHost(c->status_host);
  delete c;
  return FT_OK;
}

const char* ft_comm_last_error(ft_comm* c) { return c ? c->err.c_str() : "null communicator"; }

int ft_comm_export_fd(ft_comm* c, int* fd_out) {
  if (!c || c->mem_kind != FT_MEM_VMM || !fd_out) return fail(c, FT_ERR_INVALID_ARG, "export_fd needs a VMM heap");
  int fd = -1;
  FT_CU(c, driver().p_cuMemExportToShareableHandle(&fd, c->handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  *fd_out = fd;
  return FT_OK;
}

int ft_comm_import_fd(ft_comm* c, int peer, int fd) {
  if (!c || peer < 0 || peer >= c->world || peer == c->rank) return fail(c, FT_ERR_INVALID_ARG, "bad peer");
  FT_CUDA(c, cudaSetDevice(c->device));
  CUmemGenericAllocationHandle h = 0;
  FT_CU(c, driver().p_cuMemImportFromShareableHandle(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  CUdeviceptr va = 0;
  int rc = map_handle(c, h, c->total_bytes, &va);
  if (rc != FT_OK) return rc;
  c->peer_handle[peer] = h;
  c->peer_base[peer] = (unsigned char*)va;
  c->peer_is_vmm[peer] = true;
  return FT_OK;
}

int ft_comm_export_ipc(ft_comm* c, void* blob64) {
  if (!c || c->mem_kind != FT_MEM_IPC || !blob64) return fail(c, FT_ERR_INVALID_ARG, "export_ipc needs a cudaMalloc heap");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  FT_CUDA(c, cudaIpcGetMemHandle((cudaIpcMemHandle_t*)blob64, c->ipc_ptr));
  return FT_OK;
}

int ft_comm_import_ipc(ft_comm* c, int peer, const void* blob64) {
  if (!c || peer < 0 || peer >= c->world || peer == c->rank) return fail(c, FT_ERR_INVALID_ARG, "bad peer");
  FT_CUDA(c, cudaSetDevice(c->device));
  cudaIpcMemHandle_t h;
  std::memcpy(&h, blob64, sizeof h);
  void* p = nullptr;
  FT_CUDA(c, cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  c->peer_base[peer] = (unsigned char*)p;
  c->peer_is_ipc[peer] = true;
  return FT_OK;
}

int ft_comm_connect_local(ft_comm** comms, int n) {
  if (!comms || n < 1) return FT_ERR_INVALID_ARG;
  for (int i = 0; i < n; ++i)
    if (!comms[i] || comms[i]->world != n || comms[i]->rank != i || comms[i]->total_bytes != comms[0]->total_bytes)
      return fail(comms[i], FT_ERR_INVALID_ARG, "connect_local: communicators must be ranks 0..n-1 of one world with equal heaps");
  for (int i = 0; i < n; ++i) {
    ft_comm* c = comms[i];
    for (int j = 0; j < n; ++j) {
      if (i == j) continue;
      ft_comm* o = comms[j];
      if (o->device != c->device) {
        if (o->mem_kind == FT_MEM_VMM) {  // let c's device reach o's allocation through o's own mapping
          CUmemAccessDesc acc{};
          acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
          acc.location.id = c->device;
          acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
          FT_CU(c, driver().p_cuMemSetAccess(o->va, o->total_bytes, &acc, 1));
        } else {
          FT_CUDA(c, cudaSetDevice(c->device));
          cudaError_t e = cudaDeviceEnablePeerAccess(o->device, 0);
          if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return fail(c, FT_ERR_CUDA, cudaGetErrorString(e));
          cudaGetLastError();
        }
      }
      c->peer_base[j] = local_base(o);
    }
  }
  // NVLS for a world that lives in one process: one multicast object, every rank's device added, every
  // rank's heap bound at offset 0, one mapping per rank.  Needs VMM heaps on distinct devices that all
  // support multicast; anything else (or FT_NVLS=0) leaves the world on plain peer access.
  bool want_mc = n > 1;
  if (const char* e = std::getenv("FT_NVLS"); e && e[0] == '0') want_mc = false;
  for (int i = 0; i < n && want_mc; ++i) {
    want_mc = comms[i]->mem_kind == FT_MEM_VMM && ft_comm_mc_supported(comms[i]);
    for (int j = 0; j < i && want_mc; ++j) want_mc = comms[j]->device != comms[i]->device;
  }
  if (want_mc) {
    Driver& d = driver();
    CUmulticastObjectProp mp{};
    mp.numDevices = (unsigned)n;
    mp.size = comms[0]->total_bytes;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    CUmemGenericAllocationHandle h = 0;
    bool ok = d.p_cuMulticastCreate(&h, &mp) == CUDA_SUCCESS;
    std::shared_ptr<McOwner> owner;
    if (ok) owner = std::make_shared<McOwner>(h);
    for (int i = 0; i < n && ok; ++i) ok = d.p_cuMulticastAddDevice(h, comms[i]->device) == CUDA_SUCCESS;
    for (int i = 0; i < n && ok; ++i) {
      ft_comm* c = comms[i];
      cudaSetDevice(c->device);
      ok = d.p_cuMulticastBindMem(h, 0, c->handle, 0, c->total_bytes, 0) == CUDA_SUCCESS;
      if (!ok) break;
      c->mc_handle = h;
      c->mc_owner = owner;
      c->mc_bound = true;
      c->mc_have = true;
      ok = map_handle(c, h, c->total_bytes, &c->mc_va) == FT_OK;
    }
    if (!ok) {   // undo: a half-bound world must not claim NVLS
      for (int i = 0; i < n; ++i) {
        ft_comm* c = comms[i];
        if (c->mc_va) { d.p_cuMemUnmap(c->mc_va, c->total_bytes); d.p_cuMemAddressFree(c->mc_va, c->total_bytes); c->mc_va = 0; }
        if (c->mc_bound && d.p_cuMulticastUnbind) d.p_cuMulticastUnbind(h, c->device, 0, c->total_bytes);
        c->mc_bound = c->mc_have = false;
        c->mc_handle = 0;
        c->mc_owner.reset();
        c->err.clear();
      }
      owner.reset();
    }
  }
  for (int i = 0; i < n; ++i) {
    int rc = ft_comm_finalize(comms[i]);
    if (rc != FT_OK) return rc;
  }
  return FT_OK;
}

int ft_comm_finalize(ft_comm* c) {
  if (!c) return FT_ERR_INVALID_ARG;
  for (int r = 0; r < c->world; ++r)
    if (!c->peer_base[r]) return fail(c, FT_ERR_INVALID_ARG, "peer " + std::to_string(r) + " was never imported");
  ftk::CommDev& d = c->dev;
  std::memset(&d, 0, sizeof d);
  for (int r = 0; r < c->world; ++r) {
    d.heap[r] = c->peer_base[r];
    d.flags[r] = (unsigned long long*)(c->peer_base[r] + c->flags_off);
  }
  d.mc_heap = c->mc_bound ? (unsigned char*)c->mc_va : nullptr;
  d.call_count = c->call_count;
  d.arrived = c->arrived;
  d.status = c->status_dev;
  d.rank = c->rank;
  d.world = c->world;
  d.timeout_ns = (unsigned long long)(c->timeout_ms * 1e6);
  d.heap_bytes = c->total_bytes;
  c->finalized = true;
  // The selection policy: the calibration file named by FT_CALIBRATION, else the packaged one; without
  // either the cost model's built-in parameters decide.
  if (!c->policy) {
    c->policy = new ft_policy(c->world);
    char why[256];
    ft_policy_load(c->policy, nullptr, why, sizeof why);
  }
  if (const char* e = std::getenv("FT_ALGO"); e && *e) {
    static const char* names[] = {"auto", "staged", "oneshot", "nvls", "hybrid", "ll", "push", "", "", "nvls1"};
    for (int i = 0; i < 10; ++i)
      if (names[i][0] && !std::strcmp(e, names[i])) c->forced_algo = i;
  }
  // Device tables of the shapes a call is likely to ask for are built now, so that the first step of a
  // training loop (or a CUDA graph capture) never stops for an allocation and a synchronous upload.
  if (c->world > 1) {
    FT_CUDA(c, cudaSetDevice(c->device));
    DevPlanEntry* pe = nullptr;
    int rc = get_plan(c, ft::Shape::flat(c->world), &pe);
    if (rc == FT_OK) rc = get_plan(c, ft::Shape::make_ring(c->world), &pe);
    if (rc != FT_OK) return rc;
    for (const ft::Shape& s : c->policy->p.table_shapes())
      if (get_plan(c, s, &pe) != FT_OK) c->err.clear();   // a bad row costs nothing: the call that wants it reports
  }
  return FT_OK;
}

ft_policy* ft_comm_policy(ft_comm* c) { return c ? c->policy : nullptr; }

int ft_comm_choose(ft_comm* c, size_t count, int dtype, int op, const void* buf, ft_choice* out) {
  if (!c || !out) return FT_ERR_INVALID_ARG;
  Prepared pr;
  int dummy = 0;
  int rc = prepare(c, nullptr, buf ? (void*)buf : (void*)&dummy, count, dtype, op, &pr);
  if (rc != FT_OK) return rc;
  ft_policy_fill_choice(choose_for(c, pr), out);
  return FT_OK;
}

// ---- multicast -------------------------------------------------------------------------
int ft_comm_mc_supported(ft_comm* c) {
  if (!c || c->mem_kind != FT_MEM_VMM) return 0;
  Driver& d = driver();
  if (!d.ok || !d.p_cuMulticastCreate || !d.p_cuMulticastAddDevice || !d.p_cuMulticastBindMem) return 0;
  int mc = 0;
  if (d.p_cuDeviceGetAttribute(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, c->device) != CUDA_SUCCESS) return 0;
  return mc;
}

int ft_comm_mc_create(ft_comm* c, int* fd_out) {
  if (!ft_comm_mc_supported(c) || !fd_out) return fail(c, FT_ERR_NOT_AVAILABLE, "multicast not supported");
  CUmulticastObjectProp mp{};
  mp.numDevices = (unsigned)c->world;
  mp.size = c->total_bytes;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  FT_CU(c, driver().p_cuMulticastCreate(&c->mc_handle, &mp));
  c->mc_owner = std::make_shared<McOwner>(c->mc_handle);
  c->mc_have = true;
  int fd = -1;
  FT_CU(c, driver().p_cuMemExportToShareableHandle(&fd, c->mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  *fd_out = fd;
  return FT_OK;
}

int ft_comm_mc_join(ft_comm* c, int fd) {
  if (!ft_comm_mc_supported(c)) return fail(c, FT_ERR_NOT_AVAILABLE, "multicast not supported");
  if (fd >= 0) {
    FT_CU(c, driver().p_cuMemImportFromShareableHandle(&c->mc_handle, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
    c->mc_owner = std::make_shared<McOwner>(c->mc_handle);
    c->mc_have = true;
  }
  if (!c->mc_have) return fail(c, FT_ERR_INVALID_ARG, "no multicast object");
  FT_CU(c, driver().p_cuMulticastAddDevice(c->mc_handle, c->device));
  c->mc_joined = true;
  return FT_OK;
}

int ft_comm_mc_bind(ft_comm* c) {
  if (!c || !c->mc_joined) return fail(c, FT_ERR_INVALID_ARG, "join the multicast object first");
  FT_CU(c, driver().p_cuMulticastBindMem(c->mc_handle, 0, c->handle, 0, c->total_bytes, 0));
  c->mc_bound = true;
  int rc = map_handle(c, c->mc_handle, c->total_bytes, &c->mc_va);
  if (rc != FT_OK) return rc;
  if (c->finalized) c->dev.mc_heap = (unsigned char*)c->mc_va;
  return FT_OK;
}

int ft_comm_has_nvls(ft_comm* c) { return c && c->mc_bound && c->mc_va; }

// ---- heap ------------------------------------------------------------------------------
void* ft_comm_heap_base(ft_comm* c) { return c ? local_base(c) : nullptr; }
size_t ft_comm_heap_bytes(ft_comm* c) { return c ? c->user_bytes : 0; }
void* ft_comm_alloc(ft_comm* c, size_t bytes) {
  if (!c || !local_base(c)) return nullptr;
  const size_t off = c->heap_alloc.alloc(bytes);
  return off == ft::HeapAllocator::kNone ? nullptr : local_base(c) + off;
}
int ft_comm_free(ft_comm* c, void* p) {
  if (!c || !p) return FT_ERR_INVALID_ARG;
  const unsigned char* b = local_base(c);
  const unsigned char* q = (const unsigned char*)p;
  if (!b || q < b || q >= b + c->user_bytes || !c->heap_alloc.free((size_t)(q - b)))
    return fail(c, FT_ERR_INVALID_ARG, "ft_comm_free: not the start of a block from ft_comm_alloc");
  return FT_OK;
}
void ft_comm_alloc_reset(ft_comm* c) {
  if (!c) return;
  c->heap_alloc.reset();
  // the host pipeline's chunk buffers came from the heap too: it takes new ones on its next call
  c->hp.chunk = 0;
  for (bool& u : c->hp.used) u = false;
}
size_t ft_comm_heap_free_bytes(ft_comm* c) { return c ? c->heap_alloc.largest_free() : 0; }
int ft_comm_rank(ft_comm* c) { return c ? c->rank : -1; }
int ft_comm_world(ft_comm* c) { return c ? c->world : 0; }
int ft_comm_mem_kind(ft_comm* c) { return c ? c->mem_kind : -1; }
void ft_comm_set_timeout_ms(ft_comm* c, double ms) {
  if (!c) return;
  c->timeout_ms = ms;
  c->dev.timeout_ns = (unsigned long long)(ms * 1e6);
}
void ft_comm_set_max_lanes(ft_comm* c, int lanes) { if (c) c->max_lanes = lanes; }
void ft_comm_set_oneshot_max(ft_comm* c, size_t bytes) { if (c) c->oneshot_max = bytes; }
void ft_comm_set_hybrid(ft_comm* c, double byte_fraction, double lane_fraction) {
  if (!c) return;
  c->hybrid_fraction = byte_fraction < 0 ? 0 : (byte_fraction > 1 ? 1 : byte_fraction);
  c->hybrid_lane_fraction = lane_fraction < 0 ? 0 : (lane_fraction > 1 ? 1 : lane_fraction);
}

// ---- collectives -----------------------------------------------------------------------
int ft_allreduce(ft_comm* c, const void* sendbuf, void* recvbuf, size_t count, int dtype, int op, const int* widths,
                 int nw, int lonely, int ring, int algo, float scale, void* stream) {
  Prepared pr;
  int rc = prepare(c, sendbuf, recvbuf, count, dtype, op, &pr);
  if (rc != FT_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (count == 0) return FT_OK;
  if (c->world == 1) {  // single rank: the reference's memcpy shortcut (mpi_mod.hpp:1739-1746)
    if (sendbuf && sendbuf != recvbuf) FT_CUDA(c, cudaMemcpyAsync(recvbuf, sendbuf, pr.bytes, cudaMemcpyDeviceToDevice, st));
    // every floating type is scaled, as the kernels of larger worlds do; integer and bitwise results never are
    if (scale != 1.0f && (dtype == FT_F32 || dtype == FT_BF16 || dtype == FT_F16 || dtype == FT_F64))
      return ft_scale_inplace(dtype, recvbuf, count, scale, stream);
    return FT_OK;
  }
  ft::Shape auto_shape;
  const bool was_auto = algo == FT_ALGO_AUTO;
  const bool caller_shape = nw > 0 || ring;   // the caller (or FT_TOPO) named the plan, as opposed to the policy
  if (algo == FT_ALGO_AUTO) {
    if (nw > 0 || ring) {
      algo = FT_ALGO_STAGED;
    } else if (c->forced_algo != FT_ALGO_AUTO) {
      algo = c->forced_algo;
    } else {   // one policy for every caller: measured winner for this size, else the cost model
      const ft::PolicyChoice ch = choose_for(c, pr);
      ft_choice cc;
      ft_policy_fill_choice(ch, &cc);
      algo = cc.algo;
      const bool flat_shape = !ch.shape.ring && ch.shape.lonely == 0 && ch.shape.widths.size() <= 1;
      if (algo == FT_ALGO_STAGED || (algo == FT_ALGO_LL && !flat_shape)) {
        auto_shape = ch.shape;
        widths = auto_shape.widths.data();
        nw = (int)auto_shape.widths.size();
        lonely = auto_shape.lonely;
        ring = auto_shape.ring ? 1 : 0;
      } else if (algo == FT_ALGO_HYBRID) {
        ft_comm_set_hybrid(c, ch.hybrid_bytes, ch.hybrid_lanes);
      }
    }
  }
  // A device tensor outside the heap that is larger than one staging slot goes through the slots piecewise.
  if (!pr.heap_resident && pr.bytes > c->staging_bytes && (algo == FT_ALGO_STAGED || algo == FT_ALGO_ONESHOT)) {
    const size_t per = (c->staging_bytes / pr.es) / 64 * 64;
    if (!per) return fail(c, FT_ERR_TOO_LARGE, "staging slot smaller than 64 elements");
    const unsigned char* src = (const unsigned char*)sendbuf;
    unsigned char* dst = (unsigned char*)recvbuf;
    for (size_t lo = 0; lo < count; lo += per) {
      const size_t n = count - lo < per ? count - lo : per;
      rc = ft_allreduce(c, src ? src + lo * pr.es : nullptr, dst + lo * pr.es, n, dtype, op, widths, nw, lonely, ring,
                        FT_ALGO_STAGED, scale, stream);
      if (rc != FT_OK) return rc;
    }
    return FT_OK;
  }
  // A shape together with the low-latency protocol: the plan runs on tagged words (one NVLink trip per stage).  An
  // explicit shape under AUTO (FT_TOPO) takes that form too while the message is small enough for it to pay.
  const bool shaped = nw > 0 || ring;
  if (shaped && (algo == FT_ALGO_LL || (was_auto && caller_shape && algo == FT_ALGO_STAGED && pr.bytes <= c->ll_tree_max))) {
    const ft::Shape shape = make_shape(c->world, widths, nw, lonely, ring);
    DevPlanEntry* pe = nullptr;
    rc = get_plan(c, shape, &pe);
    if (rc != FT_OK) return rc;
    if (algo == FT_ALGO_LL || ll_tree_fits(c, pr, count, pe->nslots)) {
      c->stat_calls[FT_ALGO_LL]++;
      c->stat_bytes[FT_ALGO_LL] += pr.bytes;
      return launch_ll_tree_call(c, pr, sendbuf, recvbuf, count, shape, scale, -1, -1, 3, true, 0, st);
    }
  }
  if ((algo >= 0 && algo < 7) || algo == FT_ALGO_NVLS1) { c->stat_calls[algo]++; c->stat_bytes[algo] += pr.bytes; }
  if (algo == FT_ALGO_NVLS1) {
    if (!ft_comm_has_nvls(c)) return fail(c, FT_ERR_NOT_AVAILABLE, "NVLS multicast is not bound on this communicator");
    if (pr.pol != ftk::POL_F32 && pr.pol != ftk::POL_BF16 && pr.pol != ftk::POL_F16)
      return fail(c, FT_ERR_UNSUPPORTED_TYPE, "the switch reduces floating types only");
    if (pr.bytes > c->staging_bytes) return fail(c, FT_ERR_TOO_LARGE, "one-shot message exceeds the staging slot");
    ftk::OneShotArgs a{};
    a.slot_off = c->staging_off;
    a.user_in = sendbuf ? sendbuf : recvbuf;
    a.user_out = recvbuf;
    a.count = count;
    a.elem_size = pr.es;
    a.phase_mask = 7;
    a.user_vec_ok = (((uintptr_t)a.user_in | (uintptr_t)a.user_out) & 15) == 0;
    a.scale = scale;
    int lanes = pick_lanes(c, pr.bytes, 4096);
    if (c->nvls1_max_lanes > 0 && lanes > c->nvls1_max_lanes) lanes = c->nvls1_max_lanes;
    cudaError_t e = ftk::launch_nvls_oneshot(pr.pol, c->dev, a, c->staging_bytes, lanes, c->nvls_cfg.threads > 512 ? 512 : c->nvls_cfg.threads, st);
    if (e != cudaSuccess) return fail(c, FT_ERR_CUDA, std::string("NVLS one-shot launch: ") + cudaGetErrorString(e));
    return FT_OK;
  }
  if (algo == FT_ALGO_LL) return launch_ll_call(c, pr, sendbuf, recvbuf, count, scale, 3, true, 0, st);
  if (algo == FT_ALGO_ONESHOT) return launch_oneshot_call(c, pr, sendbuf, recvbuf, count, scale, 7, 0, st);
  if (algo == FT_ALGO_PUSH) return launch_push_call(c, pr, sendbuf, recvbuf, count, scale, true, st);
  if (algo == FT_ALGO_NVLS || algo == FT_ALGO_HYBRID) {
    if (!ft_comm_has_nvls(c)) return fail(c, FT_ERR_NOT_AVAILABLE, "NVLS multicast is not bound on this communicator");
    if (!pr.heap_resident) return fail(c, FT_ERR_INVALID_ARG, "NVLS all-reduce needs a 16-byte aligned tensor in the symmetric heap");
    if (pr.bytes % 16) return fail(c, FT_ERR_INVALID_ARG, "NVLS all-reduce needs a multiple of 16 bytes");
    if (sendbuf && sendbuf != recvbuf) FT_CUDA(c, cudaMemcpyAsync(recvbuf, sendbuf, pr.bytes, cudaMemcpyDeviceToDevice, st));
    ftk::NvlsArgs a{};
    a.work_off = (uint64_t)((unsigned char*)recvbuf - local_base(c));
    a.count = count;
    a.elem_size = pr.es;
    a.block_elems = pick_block_elems(count, c->world, pr.es);
    a.scale = scale;
    int lanes = pick_lanes(c, a.block_elems * pr.es, 8192, c->nvls_ctas_per_sm);
    if (c->nvls_max_lanes > 0 && lanes > c->nvls_max_lanes) lanes = c->nvls_max_lanes;
    cudaError_t e;
    if (algo == FT_ALGO_HYBRID && lanes >= 8) {
      // share of each block that goes through the switch, and the same share of the lanes
      const double f = c->hybrid_fraction;
      uint64_t nvls_bytes = (uint64_t)(a.block_elems * pr.es * f);
      nvls_bytes = nvls_bytes >= (64u << 10) ? nvls_bytes / 1024 * 1024 : nvls_bytes / 16 * 16;   // both parts start on a warp-request boundary
      int nvls_lanes = (int)(lanes * c->hybrid_lane_fraction + 0.5);
      if (nvls_lanes < 1) nvls_lanes = 1;
      if (nvls_lanes > lanes - 1) nvls_lanes = lanes - 1;
      e = ftk::launch_hybrid(pr.pol, c->dev, a, lanes, nvls_lanes, nvls_bytes, st);
    } else {
      a.stripe_bytes = c->nvls_stripe;
      e = ftk::launch_nvls(pr.pol, c->dev, a, lanes, 0, c->nvls_cfg, st);
    }
    if (e != cudaSuccess) return fail(c, e == cudaErrorInvalidValue ? FT_ERR_UNSUPPORTED_TYPE : FT_ERR_CUDA, std::string("NVLS launch: ") + cudaGetErrorString(e));
    return FT_OK;
  }
  return launch_staged_call(c, pr, sendbuf, recvbuf, count, make_shape(c->world, widths, nw, lonely, ring), scale, -1, -1, true, st);
}

// All-reduce of data that lives in host memory, the form the reference's entry point takes
// (mpi_mod.hpp:1723-1778 works on host buffers only).  The message is cut into chunks that travel
// through three buffers of the symmetric heap on three streams: while chunk k is being reduced over
// NVLink, chunk k+1 is on its way in over PCIe and chunk k-1 on its way out, so a large message costs
// about max(host-to-device, device-to-host) time instead of their sum plus the collective.
// Every rank has to make the call (the chunk buffers are taken from the heap on first use, which keeps
// the heaps symmetric only if every rank does it at the same point of its allocation sequence).
// Asynchronous with respect to the host for pinned buffers; ordered after what `stream` holds at the
// call, and `stream` waits for the last chunk.
void ft_comm_set_host_chunk(ft_comm* c, size_t bytes) { if (c && !c->hp.chunk) c->host_chunk_bytes = bytes < 65536 ? 65536 : bytes; }

int ft_allreduce_host(ft_comm* c, const void* host_send, void* host_recv, size_t count, int dtype, int op, const int* widths,
                      int nw, int lonely, int ring, int algo, float scale, void* stream) {
  if (!c || !c->finalized) return fail(c, FT_ERR_INVALID_ARG, "communicator not finalized");
  const size_t es = ft_dtype_size((ft_dtype)dtype);
  if (!es || ftk::policy_id(op, dtype) < 0)
    return fail(c, FT_ERR_UNSUPPORTED_TYPE, std::string("Type ") + ft_dtype_name((ft_dtype)dtype) + " is not supported");
  if (!host_recv && count) return fail(c, FT_ERR_INVALID_ARG, "recvbuf is null");
  if (count == 0) return FT_OK;
  FT_CUDA(c, cudaSetDevice(c->device));
  constexpr int D = ft_comm::HostPipe::kDepth;
  ft_comm::HostPipe& hp = c->hp;
  if (!hp.in) {
    FT_CUDA(c, cudaStreamCreateWithFlags(&hp.in, cudaStreamNonBlocking));
    FT_CUDA(c, cudaStreamCreateWithFlags(&hp.run, cudaStreamNonBlocking));
    FT_CUDA(c, cudaStreamCreateWithFlags(&hp.out, cudaStreamNonBlocking));
    FT_CUDA(c, cudaEventCreateWithFlags(&hp.start, cudaEventDisableTiming));
    for (int k = 0; k < D; ++k) {
      FT_CUDA(c, cudaEventCreateWithFlags(&hp.in_done[k], cudaEventDisableTiming));
      FT_CUDA(c, cudaEventCreateWithFlags(&hp.run_done[k], cudaEventDisableTiming));
      FT_CUDA(c, cudaEventCreateWithFlags(&hp.out_done[k], cudaEventDisableTiming));
    }
  }
  if (!hp.chunk) {   // the same arithmetic on every rank: equal heaps give equal chunk sizes and offsets
    size_t chunk = c->host_chunk_bytes;
    const size_t room = c->heap_alloc.largest_free() / D;
    if (chunk > room) chunk = room;
    chunk = chunk / 4096 * 4096;
    if (!chunk) return fail(c, FT_ERR_TOO_LARGE, "no room in the symmetric heap for the host staging chunks");
    for (int k = 0; k < D; ++k) {
      hp.slot[k] = (unsigned char*)ft_comm_alloc(c, chunk);
      if (!hp.slot[k]) return fail(c, FT_ERR_TOO_LARGE, "no room in the symmetric heap for the host staging chunks");
    }
    hp.chunk = chunk;
  }
  const size_t per = hp.chunk / es / 64 * 64;   // elements per chunk: whole 16-byte vectors for every type
  cudaStream_t user = (cudaStream_t)stream;
  FT_CUDA(c, cudaEventRecord(hp.start, user));
  FT_CUDA(c, cudaStreamWaitEvent(hp.in, hp.start, 0));
  // results of an earlier call may still be leaving a buffer on the output stream
  const unsigned char* src = (const unsigned char*)(host_send ? host_send : host_recv);
  unsigned char* dst = (unsigned char*)host_recv;
  int k = 0;
  for (size_t lo = 0; lo < count; lo += per, k = (k + 1) % D) {
    const size_t n = count - lo < per ? count - lo : per;
    if (hp.used[k]) FT_CUDA(c, cudaStreamWaitEvent(hp.in, hp.out_done[k], 0));   // the buffer's previous chunk has left
    FT_CUDA(c, cudaMemcpyAsync(hp.slot[k], src + lo * es, n * es, cudaMemcpyHostToDevice, hp.in));
    FT_CUDA(c, cudaEventRecord(hp.in_done[k], hp.in));
    FT_CUDA(c, cudaStreamWaitEvent(hp.run, hp.in_done[k], 0));
    int rc = ft_allreduce(c, nullptr, hp.slot[k], n, dtype, op, widths, nw, lonely, ring, algo, scale, hp.run);
    if (rc != FT_OK) return rc;
    FT_CUDA(c, cudaEventRecord(hp.run_done[k], hp.run));
    FT_CUDA(c, cudaStreamWaitEvent(hp.out, hp.run_done[k], 0));
    FT_CUDA(c, cudaMemcpyAsync(dst + lo * es, hp.slot[k], n * es, cudaMemcpyDeviceToHost, hp.out));
    FT_CUDA(c, cudaEventRecord(hp.out_done[k], hp.out));
    hp.used[k] = true;
  }
  for (int j = 0; j < D; ++j)
    if (hp.used[j]) FT_CUDA(c, cudaStreamWaitEvent(user, hp.out_done[j], 0));
  return FT_OK;
}

// The two halves of the staged plan as collectives of their own (in place, symmetric heap only).
static int phase_call(ft_comm* c, void* buf, size_t count, int dtype, int op, const int* widths, int nw, int lonely, int ring,
                      float scale, bool gather, void* stream) {
  Prepared pr;
  int rc = prepare(c, nullptr, buf, count, dtype, op, &pr);
  if (rc != FT_OK) return rc;
  if (count == 0) return FT_OK;
  if (c->world == 1) {
    if (!gather && scale != 1.0f && (dtype == FT_F32 || dtype == FT_BF16 || dtype == FT_F16 || dtype == FT_F64))
      return ft_scale_inplace(dtype, buf, count, scale, stream);
    return FT_OK;
  }
  DevPlanEntry* pe = nullptr;
  const ft::Shape shape = make_shape(c->world, widths, nw, lonely, ring);
  c->stat_calls[gather ? 8 : 7]++;
  c->stat_bytes[gather ? 8 : 7] += pr.bytes;
  // Flat shape on a tensor the switch can reduce: one multimem pass (ld_reduce of the own block into the own
  // buffer, or multimem.st of the own block to everyone) instead of N-1 peer loads per vector.  Block r ends up
  // on / comes from rank r, exactly as in the flat plan.
  const bool flat = !shape.ring && shape.lonely == 0 && shape.widths.size() == 1;
  // (measured, 256 MiB fp32, reduce-scatter / all-gather: 8 GPUs 0.405 / 0.405 ms through the switch against 0.465 / 0.420 ms
  //  with peer loads; 4 GPUs 0.409 / 0.405 against 0.357 / 0.352; with two ranks a multimem pass moves twice the bytes
  //  of a plain peer read - so the switch takes over from five ranks up)
  if (flat && (c->phase_nvls == 2 || (c->phase_nvls == 1 && c->world > 4)) && nvls_eligible(c, pr)) {
    ftk::NvlsArgs a{};
    a.work_off = (uint64_t)((unsigned char*)buf - local_base(c));
    a.count = count;
    a.elem_size = pr.es;
    a.block_elems = pick_block_elems(count, c->world, pr.es);
    a.scale = gather ? 1.0f : scale;
    int lanes = pick_lanes(c, a.block_elems * pr.es, 8192, c->nvls_ctas_per_sm);
    if (c->nvls_max_lanes > 0 && lanes > c->nvls_max_lanes) lanes = c->nvls_max_lanes;
    cudaError_t e = ftk::launch_nvls(pr.pol, c->dev, a, lanes, gather ? 2 : 1, c->nvls_cfg, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(c, FT_ERR_CUDA, std::string("NVLS phase launch: ") + cudaGetErrorString(e));
    return FT_OK;
  }
  rc = get_plan(c, shape, &pe);
  if (rc != FT_OK) return rc;
  const int half = pe->nstages / 2;
  return launch_staged_call(c, pr, nullptr, buf, count, shape, scale, gather ? half : 0, gather ? pe->nstages : half, true,
                            (cudaStream_t)stream, true);
}
int ft_reduce_scatter(ft_comm* c, void* buf, size_t count, int dtype, int op, const int* widths, int nw, int lonely, int ring,
                      float scale, void* stream) {
  return phase_call(c, buf, count, dtype, op, widths, nw, lonely, ring, scale, false, stream);
}
int ft_all_gather(ft_comm* c, void* buf, size_t count, int dtype, const int* widths, int nw, int lonely, int ring, void* stream) {
  // gathers move bytes; any operator the type supports selects a kernel instantiation
  const int op = ftk::policy_id(FT_SUM, dtype) >= 0 ? FT_SUM : FT_BAND;
  return phase_call(c, buf, count, dtype, op, widths, nw, lonely, ring, 1.0f, true, stream);
}
uint64_t ft_block_elems(uint64_t count, int world, int elem_size) {
  if (world < 1 || (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8)) return 0;
  return pick_block_elems(count, world, (uint32_t)elem_size);
}
uint64_t ft_comm_block_elems(ft_comm* c, size_t count, int dtype) {
  const size_t es = ft_dtype_size((ft_dtype)dtype);
  if (!c || !es) return 0;
  return pick_block_elems(count, c->world, (uint32_t)es);
}

int ft_allreduce_emulate_stage(ft_comm* c, const void* sendbuf, void* recvbuf, size_t count, int dtype, int op,
                               const int* widths, int nw, int lonely, int ring, float scale, int stage_begin,
                               int stage_end, void* stream) {
  Prepared pr;
  int rc = prepare(c, sendbuf, recvbuf, count, dtype, op, &pr);
  if (rc != FT_OK) return rc;
  if (count == 0 || c->world == 1) return FT_OK;
  return launch_staged_call(c, pr, sendbuf, recvbuf, count, make_shape(c->world, widths, nw, lonely, ring), scale,
                            stage_begin, stage_end, false, (cudaStream_t)stream);
}

int ft_allreduce_emulate_oneshot(ft_comm* c, const void* sendbuf, void* recvbuf, size_t count, int dtype, int op,
                                 float scale, int phase, uint64_t call, void* stream) {
  Prepared pr;
  int rc = prepare(c, sendbuf, recvbuf, count, dtype, op, &pr);
  if (rc != FT_OK) return rc;
  if (count == 0) return FT_OK;
  return launch_oneshot_call(c, pr, sendbuf, recvbuf, count, scale, (uint32_t)phase & 5u, call, (cudaStream_t)stream);
}

int ft_allreduce_emulate_push(ft_comm* c, void* recvbuf, size_t count, int dtype, int op, float scale, void* stream) {
  Prepared pr;
  int rc = prepare(c, nullptr, recvbuf, count, dtype, op, &pr);
  if (rc != FT_OK) return rc;
  if (count == 0 || c->world == 1) return FT_OK;
  return launch_push_call(c, pr, nullptr, recvbuf, count, scale, false, (cudaStream_t)stream);
}

int ft_allreduce_emulate_ll(ft_comm* c, const void* sendbuf, void* recvbuf, size_t count, int dtype, int op, float scale,
                            int phase, uint64_t call, void* stream) {
  Prepared pr;
  int rc = prepare(c, sendbuf, recvbuf, count, dtype, op, &pr);
  if (rc != FT_OK) return rc;
  if (count == 0) return FT_OK;
  return launch_ll_call(c, pr, sendbuf, recvbuf, count, scale, (uint32_t)phase & 3u, false, call, (cudaStream_t)stream);
}
void ft_comm_set_nvls_ctas_per_sm(ft_comm* c, int n) { if (c && n >= 1 && n <= 3) c->nvls_ctas_per_sm = n; }
int ft_comm_set_nvls_config(ft_comm* c, int threads, int unroll, int weak, int max_lanes, size_t stripe_bytes) {
  if (!c) return FT_ERR_INVALID_ARG;
  if (threads) {
    if (threads < 128 || threads > 1024 || threads % 32) return fail(c, FT_ERR_INVALID_ARG, "NVLS threads per CTA: a multiple of 32 in 128..1024");
    c->nvls_cfg.threads = threads;
  }
  if (unroll) {
    if (unroll != 2 && unroll != 4 && unroll != 8) return fail(c, FT_ERR_INVALID_ARG, "NVLS vectors in flight per thread: 2, 4 or 8");
    c->nvls_cfg.unroll = unroll;
  }
  if (weak >= 0) c->nvls_cfg.weak = weak ? 1 : 0;
  if (max_lanes >= 0) c->nvls_max_lanes = max_lanes;
  if (stripe_bytes != (size_t)-1) {
    if (stripe_bytes % 16) return fail(c, FT_ERR_INVALID_ARG, "NVLS stripe: a multiple of 16 bytes");
    c->nvls_stripe = stripe_bytes;
  }
  return FT_OK;
}
void ft_comm_set_phase_nvls(ft_comm* c, int mode) { if (c && mode >= 0 && mode <= 2) c->phase_nvls = mode; }
void ft_comm_set_nvls1_max_lanes(ft_comm* c, int lanes) { if (c && lanes >= 0) c->nvls1_max_lanes = lanes; }
int ft_allreduce_emulate_ll_tree(ft_comm* c, const void* sendbuf, void* recvbuf, size_t count, int dtype, int op,
                                 const int* widths, int nw, int lonely, int ring, float scale, int stage, int phase,
                                 uint64_t call, void* stream) {
  Prepared pr;
  int rc = prepare(c, sendbuf, recvbuf, count, dtype, op, &pr);
  if (rc != FT_OK) return rc;
  if (count == 0 || c->world == 1) return FT_OK;
  return launch_ll_tree_call(c, pr, sendbuf, recvbuf, count, make_shape(c->world, widths, nw, lonely, ring), scale, stage, stage + 1,
                             (uint32_t)phase & 3u, false, call, (cudaStream_t)stream);
}
void ft_comm_set_ll_tree_max(ft_comm* c, size_t bytes) { if (c) c->ll_tree_max = bytes < ftk::kLLMaxBytes ? bytes : ftk::kLLMaxBytes; }
void ft_comm_set_ll_max(ft_comm* c, size_t bytes) { if (c) c->ll_max = bytes < ftk::kLLMaxBytes ? bytes : ftk::kLLMaxBytes; }

int ft_plan_num_stages_for(ft_comm* c, const int* widths, int nw, int lonely, int ring) {
  DevPlanEntry* pe = nullptr;
  if (get_plan(c, make_shape(c->world, widths, nw, lonely, ring), &pe) != FT_OK) return -1;
  return pe->nstages;
}

// 1 when the library was built with -DFT_BOUNDS (the kernels check every heap range before touching it)
int ft_bounds_build(void) {
#ifdef FT_BOUNDS
  return 1;
#else
  return 0;
#endif
}
// The predicate of the checked build, callable on the host (tests exercise its failing branch here, never on a GPU)
int ft_bounds_check_host(uint64_t heap_bytes, int rank, int world, uint64_t off, uint64_t len) {
  return ftk::range_in_heap(heap_bytes, rank, world, off, len) ? 1 : 0;
}

int ft_comm_status(ft_comm* c, int* out5) {
  if (!c || !out5) return FT_ERR_INVALID_ARG;
  out5[0] = c->status_host->code; out5[1] = c->status_host->index; out5[2] = c->status_host->peer;
  out5[3] = c->status_host->lane; out5[4] = (int)c->status_host->calls;
  return c->status_host->code;
}
int ft_comm_stats(ft_comm* c, uint64_t* calls10, uint64_t* bytes10) {
  if (!c || !calls10 || !bytes10) return FT_ERR_INVALID_ARG;
  for (int i = 0; i < 10; ++i) { calls10[i] = c->stat_calls[i]; bytes10[i] = c->stat_bytes[i]; }
  return FT_OK;
}
void ft_comm_clear_status(ft_comm* c) {
  if (c) { c->status_host->code = 0; c->status_host->index = c->status_host->peer = c->status_host->lane = 0; }
}
int ft_comm_wait_probe(ft_comm* c, int peer, double timeout_ms, void* stream) {
  if (!c || !c->finalized || peer < 0 || peer >= FT_MAX_RANKS) return FT_ERR_INVALID_ARG;
  cudaError_t e = ftk::launch_wait_probe(c->dev, peer, (unsigned long long)(timeout_ms * 1e6), (cudaStream_t)stream);
  return e == cudaSuccess ? FT_OK : fail(c, FT_ERR_CUDA, cudaGetErrorString(e));
}

}  // extern "C"
