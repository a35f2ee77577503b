/* FlexTree multi-GPU communicator — C API.
 *
 * One communicator per (process, GPU, stream of use).  Each rank owns a "symmetric heap":
 * device memory that every other rank maps into its own address space (CUDA VMM
 * allocations shared as POSIX file descriptors, or cudaMalloc + CUDA IPC handles), plus
 * a flag array for rendezvous.  Collective kernels read peers' heaps directly over
 * NVLink; nothing on the data path calls NCCL or MPI.
 *
 * Set-up protocol (the bootstrap that carries handles between processes is the
 * caller's: torch.distributed in the Python package):
 *     ft_comm_create                       every rank
 *     ft_comm_export_fd / _export_ipc      every rank, handle goes to all peers
 *     ft_comm_import_fd / _import_ipc      once per peer
 *     [ft_comm_mc_create on rank 0, ft_comm_mc_join on all, barrier, ft_comm_mc_bind on all]
 *     ft_comm_finalize
 * or ft_comm_connect_local() for communicators that live in one process.
 *
 * Role in the reference: MPI_COMM_WORLD + the per-call staging buffer
 * (flextree_register_the_buffer, allreduce_over_mpi/mpi_mod.hpp:1489-1507) + the
 * MPI_Comm_split sub-communicators (:1541-1548).
 */
#ifndef FLEXTREE_COMM_H_
#define FLEXTREE_COMM_H_

#include "flextree.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ft_comm ft_comm;

enum { FT_MEM_IPC = 0, FT_MEM_VMM = 1 };
/* FT_ALGO_* are defined in ft_types.h */

/* heap_bytes: symmetric memory for user tensors (ft_comm_alloc) and internal staging.
 * staging_bytes: size of ONE staging slot (two are carved out of the heap); bounds the
 * message size of calls on tensors that do not live in the heap.
 * mem_kind: FT_MEM_VMM or FT_MEM_IPC.  The calling thread's current device must be `device`. */
int ft_comm_create(int rank, int world, int device, size_t heap_bytes, size_t staging_bytes, int mem_kind,
                   ft_comm** out);
int ft_comm_destroy(ft_comm* c);
const char* ft_comm_last_error(ft_comm* c);

int ft_comm_export_fd(ft_comm* c, int* fd_out);                 /* VMM: fd of my heap allocation */
int ft_comm_import_fd(ft_comm* c, int peer, int fd);            /* VMM: map a peer's heap */
int ft_comm_export_ipc(ft_comm* c, void* blob64);               /* IPC: 64-byte cudaIpcMemHandle_t */
int ft_comm_import_ipc(ft_comm* c, int peer, const void* blob64);
/* communicators of one process (any mix of devices, or several ranks on one device for
 * single-GPU emulation): map each other directly, then finalize all of them */
int ft_comm_connect_local(ft_comm** comms, int n);
int ft_comm_finalize(ft_comm* c);
/* The communicator's selection policy (created by ft_comm_finalize from $FT_CALIBRATION or the packaged
 * calibration file; owned by the communicator).  ft_policy_load / ft_policy_add_row on it change what
 * FT_ALGO_AUTO picks. */
ft_policy* ft_comm_policy(ft_comm* c);
/* what FT_ALGO_AUTO would run for `count` elements of `dtype` at `buf` (NULL: a tensor outside the heap) */
int ft_comm_choose(ft_comm* c, size_t count, int dtype, int op, const void* buf, ft_choice* out);

/* NVLS multicast (optional; VMM heaps only) */
int ft_comm_mc_supported(ft_comm* c);
int ft_comm_mc_create(ft_comm* c, int* fd_out);                 /* one rank creates the multicast object */
int ft_comm_mc_join(ft_comm* c, int fd);                        /* fd < 0: the creator joins its own object */
int ft_comm_mc_bind(ft_comm* c);                                /* after EVERY rank has joined */
int ft_comm_has_nvls(ft_comm* c);

/* symmetric heap */
void* ft_comm_heap_base(ft_comm* c);
size_t ft_comm_heap_bytes(ft_comm* c);       /* bytes available to ft_comm_alloc */
/* `bytes` of the heap, 256-byte aligned: first fit at the lowest free offset, so every rank gets the
 * same offset provided every rank issues the same sequence of ft_comm_alloc / ft_comm_free calls (a run
 * of allocations alone comes out back to back from offset 0); NULL when no free block is large enough */
void* ft_comm_alloc(ft_comm* c, size_t bytes);
/* give a block back (p as returned by ft_comm_alloc); neighbouring free blocks merge */
int ft_comm_free(ft_comm* c, void* p);
void ft_comm_alloc_reset(ft_comm* c);          /* forget every allocation */
size_t ft_comm_heap_free_bytes(ft_comm* c);    /* largest block ft_comm_alloc could return now */
int ft_comm_rank(ft_comm* c);
int ft_comm_world(ft_comm* c);
int ft_comm_mem_kind(ft_comm* c);

/* tuning knobs */
void ft_comm_set_timeout_ms(ft_comm* c, double ms);             /* bound of every device-side wait */
void ft_comm_set_max_lanes(ft_comm* c, int lanes);              /* CTAs per collective kernel (<= 512) */

/* All-reduce of `count` elements.  recvbuf inside the symmetric heap: in place, zero copy
 * (sendbuf must be NULL or == recvbuf).  Otherwise the input is staged through the
 * internal slots and the result lands in recvbuf (count * size <= staging_bytes).
 * shape: (widths, nw, lonely, ring) as in flextree.h; nw == 0 means flat.
 * algo: FT_ALGO_*; AUTO asks the communicator's selection policy (ft_comm_policy: the measured winner for
 * this world and message size from the calibration file, else the NVSwitch cost model), unless a shape is
 * given, which selects the staged plan.  A device tensor outside the heap that exceeds one staging slot is
 * reduced piecewise.
 * scale: multiplied into floating-point results (1/world for averaging).
 * Asynchronous on `stream`; errors of device-side waits surface in ft_comm_status. */
int ft_allreduce(ft_comm* c, const void* sendbuf, void* recvbuf, size_t count, int dtype, int op, const int* widths,
                 int nw, int lonely, int ring, int algo, float scale, void* stream);
void ft_comm_set_oneshot_max(ft_comm* c, size_t bytes);
/* All-reduce of host memory (pinned for full speed): host_send (NULL: in place) -> host_recv.  The message is
 * pipelined through three chunk buffers of the symmetric heap on internal streams, so the host-to-device copy of
 * chunk k+1, the NVLink all-reduce of chunk k and the device-to-host copy of chunk k-1 overlap.  Collective:
 * every rank calls it (the chunk buffers are allocated from the heap on the first call).  Ordered after the work
 * already in `stream`; `stream` waits for the last chunk, so synchronising it completes the call.
 * ft_comm_set_host_chunk sets the chunk size (default 32 MiB) before the first such call. */
int ft_allreduce_host(ft_comm* c, const void* host_send, void* host_recv, size_t count, int dtype, int op,
                      const int* widths, int nw, int lonely, int ring, int algo, float scale, void* stream);
void ft_comm_set_host_chunk(ft_comm* c, size_t bytes);
/* The two halves of the staged all-reduce as collectives of their own (the reference runs them
 * only back to back inside tree_allreduce, mpi_mod.hpp:1550-1599 and :1620-1647).  Both work in
 * place on a buffer inside the symmetric heap, cut into `world` blocks of
 * B = ft_comm_block_elems(c, count, dtype) elements: block b = [b*B, min((b+1)*B, count)).
 *   ft_reduce_scatter  runs the reduce-scatter stages of the shape's plan: afterwards block b is
 *                      complete (and scaled) on the rank ft_plan_rs_holders names for it; every
 *                      other part of the buffer holds inputs or partial sums.
 *   ft_all_gather      runs the all-gather stages: it takes each rank's own blocks as final and
 *                      leaves every rank with every block.
 * ft_reduce_scatter followed by ft_all_gather on the same buffer and shape equals ft_allreduce
 * with FT_ALGO_STAGED.  Each call closes with a rendezvous of all ranks, so the buffer may be
 * rewritten as soon as the call has completed on the caller's stream.
 * With the flat shape, on a float tensor of a multiple of 16 bytes, NVLS multicast bound and five or more ranks, each half is one
 * multimem pass through the switch: multimem.ld_reduce of block `rank` into the own buffer (reduce-scatter),
 * multimem.st of block `rank` to every rank (all-gather). */
int ft_reduce_scatter(ft_comm* c, void* buf, size_t count, int dtype, int op, const int* widths, int nw, int lonely,
                      int ring, float scale, void* stream);
int ft_all_gather(ft_comm* c, void* buf, size_t count, int dtype, const int* widths, int nw, int lonely, int ring,
                  void* stream);
uint64_t ft_comm_block_elems(ft_comm* c, size_t count, int dtype);
/* the same without a communicator: elements per block for `count` elements of `elem_size` bytes on `world` ranks */
uint64_t ft_block_elems(uint64_t count, int world, int elem_size);
/* FT_ALGO_HYBRID: fraction of every block reduced inside the switch (the rest goes over peer
 * loads at the same time) and fraction of the kernel's CTAs given to that part */
void ft_comm_set_hybrid(ft_comm* c, double byte_fraction, double lane_fraction);

/* Single-GPU emulation helper: run only stages [stage_begin, stage_end) of the plan with no
 * rendezvous (the caller serialises ranks and stages on one stream). */
int ft_allreduce_emulate_stage(ft_comm* c, const void* sendbuf, void* recvbuf, size_t count, int dtype, int op,
                               const int* widths, int nw, int lonely, int ring, float scale, int stage_begin,
                               int stage_end, void* stream);
/* reduce+push emulation: launch rank after rank on one stream (each rank's kernel is self-contained) */
int ft_allreduce_emulate_push(ft_comm* c, void* recvbuf, size_t count, int dtype, int op, float scale, void* stream);
/* low-latency push emulation: phase 1 = push (all ranks first), phase 2 = receive and reduce */
int ft_allreduce_emulate_ll(ft_comm* c, const void* sendbuf, void* recvbuf, size_t count, int dtype, int op, float scale,
                            int phase, uint64_t call, void* stream);
/* A plan on tagged words: FT_ALGO_LL together with a shape runs that plan (tree, lonely layout, ring) with the
 * low-latency protocol - every edge of a stage is a push of {data, tag} words into a receive slot of the destination, so
 * a stage costs one one-way NVLink trip and no rendezvous (messages up to 256 KiB whose slots fit the receive area).
 * FT_ALGO_AUTO with a shape takes this form up to ft_comm_set_ll_tree_max bytes (default 64 KiB), the staged kernel above.
 * Emulation on one GPU: per stage, phase 1 (push) for every rank, then phase 2 (receive) for every rank. */
int ft_allreduce_emulate_ll_tree(ft_comm* c, const void* sendbuf, void* recvbuf, size_t count, int dtype, int op,
                                 const int* widths, int nw, int lonely, int ring, float scale, int stage, int phase,
                                 uint64_t call, void* stream);
void ft_comm_set_ll_tree_max(ft_comm* c, size_t bytes);
/* largest message AUTO sends through the low-latency push protocol (<= 256 KiB) */
void ft_comm_set_ll_max(ft_comm* c, size_t bytes);
/* CTAs per SM of the NVLS kernels (1..3, default 1) */
void ft_comm_set_nvls_ctas_per_sm(ft_comm* c, int n);
/* Launch shape of the NVLS kernels.  threads per CTA (multiple of 32 in 128..1024; 0 keeps), 16-byte vectors in
 * flight per thread (2, 4, 8; 0 keeps), weak: 1 = multimem.*.weak, 0 = .relaxed.sys (< 0 keeps), max_lanes: cap on
 * the CTAs of one launch (0 = one per SM; < 0 keeps), stripe_bytes: all-reduce ownership, 0 = rank r reduces block r,
 * else stripes of this size dealt round-robin ((size_t)-1 keeps). */
int ft_comm_set_nvls_config(ft_comm* c, int threads, int unroll, int weak, int max_lanes, size_t stripe_bytes);
/* FT_ALGO_NVLS1, one-shot through the switch: every rank publishes its input in its staging slot, one rendezvous, every
 * rank reduces the whole message with multimem.ld_reduce into recvbuf.  Any float tensor (heap or not) up to one staging
 * slot; needs NVLS.  ft_comm_set_nvls1_max_lanes caps its CTAs (default 64; 0 = one per SM). */
void ft_comm_set_nvls1_max_lanes(ft_comm* c, int lanes);
/* ft_reduce_scatter / ft_all_gather through the multimem kernels (flat shape, eligible tensor): 0 never, 1 where it
 * measured faster than peer loads (five ranks and more; the default), 2 whenever possible */
void ft_comm_set_phase_nvls(ft_comm* c, int mode);
/* one-shot emulation: phase 1 = publish input (all ranks first), phase 4 = reduce */
int ft_allreduce_emulate_oneshot(ft_comm* c, const void* sendbuf, void* recvbuf, size_t count, int dtype, int op,
                                 float scale, int phase, uint64_t call, void* stream);

/* Debugging build (python -m allreduce_over_mpi_b200.build --bounds -> lib/libflextree_bounds.so, loaded with
 * FT_LIB=bounds): the collective kernels test every run of heap bytes against the heap size before touching it; a
 * run that leaves the heap is skipped and reported as FT_ERR_BOUNDS through ft_comm_status.  ft_bounds_build says
 * which build this is; ft_bounds_check_host evaluates the same predicate on the host. */
int ft_bounds_build(void);
int ft_bounds_check_host(uint64_t heap_bytes, int rank, int world, uint64_t off, uint64_t len);

/* status block written by kernels whose bounded wait ran out: out[0..4] =
 * {ft_status, rendezvous index, peer, lane, calls completed}.  Synchronises nothing: call
 * after the stream is idle.  ft_comm_clear_status resets it. */
int ft_comm_status(ft_comm* c, int* out5);
/* usage so far, counted on the host at launch: calls and message bytes per algorithm, index FT_ALGO_STAGED ..
 * FT_ALGO_PUSH as resolved (index 0 stays empty), 7 = ft_reduce_scatter, 8 = ft_all_gather, 9 = FT_ALGO_NVLS1; ten entries each */
int ft_comm_stats(ft_comm* c, uint64_t* calls10, uint64_t* bytes10);
void ft_comm_clear_status(ft_comm* c);
/* launches a kernel that waits `timeout_ms` for a signal from `peer` that never comes */
int ft_comm_wait_probe(ft_comm* c, int peer, double timeout_ms, void* stream);

/* fd passing between processes of one node over abstract unix sockets */
int ft_fd_listen(const char* name);                                   /* -> listening socket or -1 */
int ft_fd_send(const char* name, int fd_to_send, int tag, int timeout_ms);   /* 0 on success */
int ft_fd_recv(int listen_sock, int* tag_out, int timeout_ms);        /* -> received fd or -1 */
void ft_fd_close(int fd);

#ifdef __cplusplus
}
#endif
#endif /* FLEXTREE_COMM_H_ */
