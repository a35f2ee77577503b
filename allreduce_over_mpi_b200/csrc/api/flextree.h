/* FlexTree for B200 — C API of libflextree.so.
 *
 * Three groups of entry points:
 *   1. planner / cost model / CPU executors (pure host, usable without a GPU);
 *   2. single-GPU n-way reduction kernels (ft_reduce_nway*);
 *   3. multi-GPU communicator over NVLink peer memory (ft_comm_*), in flextree_comm.h.
 *
 * Tree shapes are passed as (widths, nw, lonely, ring): bottom-up level widths whose
 * product plus `lonely` equals the world size; ring != 0 selects the ring schedule.
 * Functions that return text write a NUL-terminated string into (buf, cap) and return
 * the number of bytes needed (excluding NUL); a return >= cap means it was truncated.
 */
#ifndef FLEXTREE_H_
#define FLEXTREE_H_

#include "ft_types.h"

#ifdef __cplusplus
extern "C" {
#endif

const char* ft_version(void);

/* ---- factorisation tools (reference: cost_model/GetPrimeFactor.h, IsPrimeNumber.h,
 *      GetWidth.h, ChooseWidth.h, PrintTreeStructure.h; topo_count/factor_count.py) ---- */
int ft_prime_factors(int n, int* out, int cap);
int ft_is_prime(int n);       /* mathematical: 1 is not prime */
int ft_is_prime_loose(int n); /* the reference's predicate: 1 counts as prime */
uint64_t ft_count_ordered_factorizations(int n);
/* one shape per line, "2*2*2\n2*4\n...": legacy != 0 uses the divisor-tuple enumerator */
size_t ft_candidate_shapes(int n, int legacy, char* buf, size_t cap);
/* one candidate per line with "+1" / "-1" suffixes */
size_t ft_choose_width(int world, char* buf, size_t cap);

/* ---- cost models ---- */
double ft_cost_v0(const int* widths, int nw, int n, double chunk);
/* arg-min over ft_candidate_shapes(n); returns number of widths written, cost in *cost,
 * number of candidates scored in *ncand */
int ft_choose_v0(int n, double chunk, int* widths, int cap, double* cost, uint64_t* ncand);

typedef struct ft_v1_params {
  double launch_us, sync_us, link_gbs, hbm_gbs, stage_floor_us, nvls_gbs, oneshot_max_bytes;
  double ll_us, ll_max_bytes, push_gain;
  double peer_eff[FT_MAX_RANKS + 1];
} ft_v1_params;
void ft_v1_defaults(ft_v1_params* p);
double ft_cost_v1(int world, const int* widths, int nw, int lonely, int ring, uint64_t bytes, const ft_v1_params* p);
double ft_cost_v1_oneshot(int world, uint64_t bytes, const ft_v1_params* p);
double ft_cost_v1_nvls(int world, uint64_t bytes, const ft_v1_params* p);
/* writes the winning shape; algo_out receives "staged", "oneshot", "nvls", "ll" or "push" */
int ft_pick_algorithm(int world, uint64_t bytes, const ft_v1_params* p, int allow_oneshot, int allow_nvls,
                      int* widths, int cap, int* lonely, int* ring, char* algo_out, size_t algo_cap, double* us);
/* same with the heap condition separate: allow_push != 0 admits the in-place reduce+push kernel */
int ft_pick_algorithm2(int world, uint64_t bytes, const ft_v1_params* p, int allow_oneshot, int allow_nvls, int allow_push,
                       int* widths, int cap, int* lonely, int* ring, char* algo_out, size_t algo_cap, double* us);
/* every executable shape for `world`, one per line ("2*4", "2*2+1", "ring8") */
size_t ft_executable_shapes(int world, char* buf, size_t cap);

/* ---- selection policy: calibration table + cost model -> algorithm and shape per message size.
 * The one place where that choice is made: ft_allreduce(FT_ALGO_AUTO), MPI_Allreduce_FT, ft_bench and the
 * Python front end all go through it.  A policy is built for one world size. ---- */
typedef struct ft_policy ft_policy;
typedef struct ft_choice {
  int algo;            /* FT_ALGO_STAGED .. FT_ALGO_PUSH, FT_ALGO_NVLS1 */
  int nw;              /* shape of the plan (FT_ALGO_STAGED); flat for the others */
  int widths[16];
  int lonely, ring;
  int from_table;      /* 1: a measured winner, 0: the cost model (or the small-message default) */
  double hybrid_bytes, hybrid_lanes;   /* FT_ALGO_HYBRID: share of each block / of the CTAs that goes through the switch */
  char algo_name[16];
} ft_choice;
ft_policy* ft_policy_create(int world);
void ft_policy_destroy(ft_policy* p);
/* where ft_policy_load(path = NULL) looks: $FT_CALIBRATION, else parallel/calibration_b200.json beside the library */
size_t ft_policy_default_path(char* buf, size_t cap);
/* reads {"params": {...}, "table": {"<world>": [[bytes, algo, shape, ...], ...]}}; returns FT_OK, or
 * FT_ERR_NOT_AVAILABLE with the reason in err (the policy then keeps what it had: the built-in model) */
int ft_policy_load(ft_policy* p, const char* path, char* err, size_t err_cap);
int ft_policy_set_params(ft_policy* p, const ft_v1_params* k);
int ft_policy_get_params(ft_policy* p, ft_v1_params* k);
void ft_policy_clear_rows(ft_policy* p);
int ft_policy_num_rows(ft_policy* p);
/* one measured winner; algo as in the calibration file ("ll", "oneshot", "staged", "push", "nvls",
 * "nvls1", "hybrid-<bytes>-<lanes>"), shape as text ("8", "2*4", "2*3+1", "ring8") */
int ft_policy_add_row(ft_policy* p, uint64_t bytes, const char* algo, const char* shape);
/* in_heap: 16-byte aligned tensor inside the symmetric heap; nvls_ok: multicast bound and the message
 * qualifies (float type, multiple of 16 bytes); staging_bytes: one staging slot; ll_auto_max: below it the
 * low-latency protocol is the default where neither table nor model speaks; nvls1_ok: multicast bound and a float
 * type (the one-shot form through the switch stages any tensor through the slots) */
int ft_policy_choose(ft_policy* p, uint64_t bytes, int in_heap, int nvls_ok, uint64_t staging_bytes, uint64_t ll_auto_max,
                     int nvls1_ok, ft_choice* out);

/* ---- configuration (reference: get_stages, mpi_mod.hpp:1419-1486) ---- */
/* returns FT_OK or FT_ERR_INVALID_TOPO (message in err) */
int ft_parse_topo(const char* topo, const char* lonely_str, int world, int* widths, int cap, int* nw, int* lonely,
                  int* ring, int* is_auto, char* err, size_t err_cap);

/* ---- planner ---- */
int ft_validate_shape(int world, const int* widths, int nw, int lonely, int ring, char* err, size_t err_cap);
/* static race check of the in-place schedule; FT_OK or FT_ERR_INVALID_TOPO + message */
int ft_plan_check(int world, const int* widths, int nw, int lonely, int ring, char* err, size_t err_cap);
int ft_plan_num_stages(int world, const int* widths, int nw, int lonely, int ring);
int ft_plan_max_fanin(int world, const int* widths, int nw, int lonely, int ring);
/* elements moved between ranks by the whole schedule; 2*(world-1)*count for every valid shape */
uint64_t ft_plan_traffic(int world, const int* widths, int nw, int lonely, int ring, uint64_t count,
                         uint64_t block_elems);
size_t ft_plan_describe(int world, const int* widths, int nw, int lonely, int ring, int rank, uint64_t count,
                        uint64_t block_elems, char* buf, size_t cap);
/* builds `rank`'s device table for the shape and checks every descriptor the kernels will follow
 * (indices, block ids, fan-in, source ranks, rendezvous coverage); the communicator runs the same
 * check before it uploads a plan.  FT_OK, or FT_ERR_INVALID_TOPO with the reason in err */
int ft_dev_plan_check(int world, const int* widths, int nw, int lonely, int ring, int rank, char* err, size_t err_cap);
/* machine-readable plan: JSON {"world":..,"stages":..,"ranks":[[{"rs":1,"sync":[..],"pulls":[[block,reduce,[srcs]],..]},..],..]} */
size_t ft_plan_json(int world, const int* widths, int nw, int lonely, int ring, char* buf, size_t cap);

/* one line with the per-call quantities the reference keeps in FlexTree_Context and prints with
 * show_context() (mpi_mod.hpp:776-801): "num_nodes=.., node_label=.., num_lonely=.., data_size=..,
 * num_split=.., split_size=.., data_size_aligned=.., type_size=.., has_lonely=..".
 * MPI_Allreduce_FT prints it to stderr on every call when FT_DEBUG=1 (or higher) is set.  FT_DEBUG=2 also runs the
 * call as its two halves and prints, per rank, the first 100 values after the reduce-scatter ("Med CHECK") and after
 * the all-gather ("Tail CHECK"), the reference's data dumps (mpi_mod.hpp:1601-1613, :1657-1670). */
size_t ft_context_describe(int world, int rank, int lonely, uint64_t count, int dtype, char* buf, size_t cap);

/* ---- CPU reductions and executors ---- */
int ft_cpu_reduce(int op, int dtype, const void* const* src, void* dst, int n, size_t len, int threads);
/* all ranks in the calling thread, in place on bufs[rank] */
int ft_run_plan_snapshot(int world, const int* widths, int nw, int lonely, int ring, int op, int dtype,
                         void* const* bufs, uint64_t count, uint64_t block_elems);
/* one phase alone: stages [stage_begin, stage_end) of the plan (stage_end < 0: to the end);
 * [0, S/2) is the reduce-scatter half, [S/2, S) the all-gather half, S = ft_plan_num_stages */
int ft_run_plan_snapshot_range(int world, const int* widths, int nw, int lonely, int ring, int op, int dtype,
                               void* const* bufs, uint64_t count, uint64_t block_elems, int stage_begin, int stage_end);
/* holders[b] (b < world) = bit mask of the ranks whose block b is complete after the
 * reduce-scatter half alone; world <= 64 */
int ft_plan_rs_holders(int world, const int* widths, int nw, int lonely, int ring, uint64_t* holders);

/* thread-per-rank world: every rank thread calls ft_cpu_allreduce with the same shape */
typedef struct ft_cpu_world ft_cpu_world;
ft_cpu_world* ft_cpu_world_create(int world, double timeout_s);
void ft_cpu_world_destroy(ft_cpu_world* w);
/* fault_kind: 0 none, 1 never-signal, 2 wrong-epoch, 3 leave-early (applies when fault_rank == rank).
 * status_out[0..2] = {ft_status, rendezvous index, peer}.  Returns status_out[0]. */
int ft_cpu_allreduce(ft_cpu_world* w, int rank, const int* widths, int nw, int lonely, int ring, int op, int dtype,
                     const void* sendbuf, void* recvbuf, uint64_t count, uint64_t block_elems, int fault_kind,
                     int fault_rank, int fault_stage, int* status_out);
/* one half of the plan as a call of its own, in place on buf: phase 1 = reduce-scatter stages,
 * 2 = all-gather stages; closes with a rendezvous of all ranks (the host twin of
 * ft_reduce_scatter / ft_all_gather in flextree_comm.h, same rendezvous numbering) */
int ft_cpu_phase(ft_cpu_world* w, int rank, const int* widths, int nw, int lonely, int ring, int op, int dtype, void* buf,
                 uint64_t count, uint64_t block_elems, int phase, int* status_out);

/* ---- process-per-rank world: the ranks are ordinary processes of one host (launched like an MPI job), they
 * meet in a POSIX shared-memory segment named after `session` (unique per job) that carries control state
 * only, and pull blocks straight out of each other's buffers with process_vm_readv.  Same plans, same
 * rendezvous protocol and the same bounded waits as the thread world. */
typedef struct ft_proc_world ft_proc_world;
/* collective over the `world` processes; NULL (reason in err) if the others do not arrive within timeout_s */
ft_proc_world* ft_proc_world_join(const char* session, int rank, int world, double timeout_s, char* err, size_t err_cap);
void ft_proc_world_leave(ft_proc_world* w);
int ft_proc_world_rank(ft_proc_world* w);
int ft_proc_world_size(ft_proc_world* w);
int ft_proc_barrier(ft_proc_world* w);
const char* ft_proc_last_error(ft_proc_world* w);
/* one half alone, in place: phase 1 = reduce-scatter stages, 2 = all-gather stages (see ft_cpu_phase) */
int ft_proc_phase(ft_proc_world* w, const int* widths, int nw, int lonely, int ring, int op, int dtype, void* buf,
                  uint64_t count, int phase, int* status_out);
/* Symmetric heap of the process world (the host twin of the GPU communicator's): ft_proc_heap_create is
 * collective and gives every rank one shared segment of `bytes` that all the others map; a buffer from
 * ft_proc_alloc is reduced in place with plain loads from the peers' mappings - no system call, no copy -
 * provided every rank allocates in the same order (ft_proc_heap_symmetric checks one pointer, collectively). */
int ft_proc_heap_create(ft_proc_world* w, size_t bytes);
void* ft_proc_alloc(ft_proc_world* w, size_t bytes);
int ft_proc_free(ft_proc_world* w, void* p);
int ft_proc_heap_symmetric(ft_proc_world* w, const void* p);
/* every rank calls it with the same shape and count; in place when sendbuf is NULL or == recvbuf.
 * status_out[0..2] = {ft_status, rendezvous index, peer} */
int ft_proc_allreduce(ft_proc_world* w, const int* widths, int nw, int lonely, int ring, int op, int dtype,
                      const void* sendbuf, void* recvbuf, uint64_t count, int* status_out);

/* ---- single-GPU n-way reduction (reference: vector_add/reduce_sum_gpu.h) ---- */
/* dst[i] = src[0][i] (op) ... (op) src[n-1][i], n in [1, FT_MAX_FANIN]; src/dst are device
 * pointers, `stream` a cudaStream_t.  variant: 0 auto, 1 vector loads, 2 TMA bulk pipeline.
 * Returns ft_status; CUDA launch errors map to FT_ERR_CUDA (see ft_last_cuda_error). */
int ft_reduce_nway(int op, int dtype, const void* const* src, void* dst, int n, size_t len, int variant,
                   void* stream);
/* out = scale * sum(src) with fp32 accumulation, optionally converting fp32 inputs to a
 * bf16 result (the cast/scale epilogue used for gradient averaging).  in_dtype FT_F32 or
 * FT_BF16; out_dtype FT_F32 or FT_BF16. */
int ft_reduce_nway_scaled(int in_dtype, int out_dtype, const void* const* src, void* dst, int n, size_t len,
                          float scale, void* stream);
/* buf[i] *= scale in place for FT_F32 / FT_F64 / FT_BF16 / FT_F16 (16-bit floats through fp32, one rounding) */
int ft_scale_inplace(int dtype, void* buf, size_t len, float scale, void* stream);
const char* ft_last_cuda_error(void);

/* ---- n-way reductions of vectors in host memory, pipelined through one GPU (reference: the copy in / kernel /
 *      copy out sequence of vector_add/vector_add.cu:81-136, done there one after the other) ----
 * A pipeline owns three streams and a ring of 3 x (max_in + max_out) device chunks of chunk_bytes.
 * ft_host_pipe_reduce computes, for every j < n_out, host_dst[j][i] = host_src[0][i] (op) ... (op)
 * host_src[fanin[j]-1][i] over i < len: the inputs are copied in once per chunk and shared by all outputs; the
 * copy in of chunk k+1, the reductions of chunk k and the copy out of chunk k-1 run at the same time.
 * Host buffers should be pinned (cudaHostAlloc / cudaHostRegister), else the copies serialise.  Ordered
 * after the work in `stream`; `stream` waits for the last chunk, so synchronising it completes the call. */
typedef struct ft_host_pipe ft_host_pipe;
int ft_host_pipe_create(int device, size_t chunk_bytes, int max_in, int max_out, ft_host_pipe** out);
void ft_host_pipe_destroy(ft_host_pipe* p);
const char* ft_host_pipe_last_error(ft_host_pipe* p);
int ft_host_pipe_reduce(ft_host_pipe* p, int op, int dtype, const void* const* host_src, int n_in, const int* fanin,
                        void* const* host_dst, int n_out, size_t len, void* stream);
/* number of kernels launched by this library in this process (all entry points) */
uint64_t ft_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* FLEXTREE_H_ */
