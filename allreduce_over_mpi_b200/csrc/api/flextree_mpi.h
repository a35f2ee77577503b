/* MPI_Allreduce-compatible entry point of FlexTree.
 *
 *     int MPI_Allreduce_FT(const void* sendbuf, void* recvbuf, int count,
 *                          FT_Datatype datatype, FT_Op op, FT_Comm comm);
 *
 * Same argument order and semantics as MPI_Allreduce / the reference's MPI_Allreduce_FT
 * (allreduce_over_mpi/mpi_mod.hpp:1723-1778): FT_IN_PLACE as sendbuf reduces in place, a
 * world of one rank is a memcpy, the tree shape comes from the environment variables
 * FT_TOPO ("w0,w1,..." bottom-up, any 1 => ring, unset => flat; "auto" => cost model) and
 * FT_LONELY, read on every call.  Returns 0 on success.  Where the reference prints a
 * message and calls exit(1) (unsupported type / op, invalid FT_TOPO) this returns a
 * non-zero ft_status after printing the same message to stderr.
 *
 * A communicator is either
 *   - one rank of a thread world (ranks are threads of this process; host buffers), or
 *   - a GPU communicator (ft_comm): device buffers are reduced by the NVLink kernels on
 *     `stream`; host buffers are staged through the GPU.
 *
 * Define FLEXTREE_MPI_NAMES before including this header, in a program that does NOT include
 * a real <mpi.h>, to get the MPI spellings (MPI_Comm, MPI_FLOAT, MPI_SUM, MPI_IN_PLACE,
 * MPI_Allreduce -> MPI_Allreduce_FT, ...) so that code written against MPI compiles as is.
 */
#ifndef FLEXTREE_MPI_H_
#define FLEXTREE_MPI_H_

#include "flextree.h"
#include "flextree_comm.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ft_mpi_comm* FT_Comm;
typedef int FT_Datatype;
typedef int FT_Op;

#define FT_IN_PLACE ((const void*)(uintptr_t)1)

/* datatype handles: the reference's eleven (mpi_mod.hpp:1365-1375) plus four extensions */
#define FT_UINT8_T ((FT_Datatype)FT_U8)
#define FT_INT8_T ((FT_Datatype)FT_I8)
#define FT_UINT16_T ((FT_Datatype)FT_U16)
#define FT_INT16_T ((FT_Datatype)FT_I16)
#define FT_INT32_T ((FT_Datatype)FT_I32)
#define FT_INT64_T ((FT_Datatype)FT_I64)
#define FT_FLOAT ((FT_Datatype)FT_F32)
#define FT_DOUBLE ((FT_Datatype)FT_F64)
#define FT_C_BOOL ((FT_Datatype)FT_BOOL)
#define FT_LONG_LONG_INT ((FT_Datatype)FT_I64)
#define FT_LONG_LONG ((FT_Datatype)FT_I64)
#define FT_UINT32_T ((FT_Datatype)FT_U32)
#define FT_UINT64_T ((FT_Datatype)FT_U64)
#define FT_BFLOAT16 ((FT_Datatype)FT_BF16)
#define FT_FLOAT16 ((FT_Datatype)FT_F16)
#define FT_OP_SUM ((FT_Op)FT_SUM)
#define FT_OP_BAND ((FT_Op)FT_BAND)
#define FT_OP_MAX_UNSUPPORTED ((FT_Op)100) /* any other operator: rejected with "Unsupported op" */

/* communicators */
FT_Comm ft_mpi_thread_rank(ft_cpu_world* world, int rank);     /* rank of a thread world */
FT_Comm ft_mpi_from_comm(ft_comm* comm, void* stream);         /* GPU communicator on a CUDA stream */
FT_Comm ft_mpi_proc_rank(ft_proc_world* world);                /* this process as a rank of a process world */
/* Process world from the launcher's environment: rank / size from FT_RANK / FT_WORLD (else RANK / WORLD_SIZE,
 * what torch.distributed.run sets), session from FT_SESSION (else MASTER_PORT).  NULL on failure
 * (ft_mpi_last_error).  The counterpart of MPI_Init + MPI_COMM_WORLD for a job started as N processes. */
FT_Comm ft_mpi_proc_init_env(double timeout_s);
/* leaves the process world of a communicator made by ft_mpi_proc_init_env (MPI_Finalize) and frees it */
void ft_mpi_proc_finalize(FT_Comm c);
/* the process world behind a communicator (for ft_proc_heap_create / ft_proc_alloc), or NULL */
ft_proc_world* ft_mpi_proc_world(FT_Comm c);
int FT_Barrier(FT_Comm c);                                      /* thread and process worlds */
void ft_mpi_comm_free(FT_Comm c);
int FT_Comm_size(FT_Comm c, int* size);
int FT_Comm_rank(FT_Comm c, int* rank);
int FT_Type_size(FT_Datatype t, int* size);
int FT_Type_get_name(FT_Datatype t, char* name, int* len);

int MPI_Allreduce_FT(const void* sendbuf, void* recvbuf, int count, FT_Datatype datatype, FT_Op op, FT_Comm comm);
/* same with a 64-bit count */
int MPI_Allreduce_FT_c(const void* sendbuf, void* recvbuf, size_t count, FT_Datatype datatype, FT_Op op, FT_Comm comm);
/* prints "FlexTree enabled" (the reference's FT_enabled(), mpi_mod.hpp:8-12) */
void FT_enabled(void);
const char* ft_mpi_last_error(void);

#ifdef __cplusplus
}
#endif

#ifdef FLEXTREE_MPI_NAMES
typedef FT_Comm MPI_Comm;
typedef FT_Datatype MPI_Datatype;
typedef FT_Op MPI_Op;
#define MPI_IN_PLACE FT_IN_PLACE
#define MPI_UINT8_T FT_UINT8_T
#define MPI_INT8_T FT_INT8_T
#define MPI_UINT16_T FT_UINT16_T
#define MPI_INT16_T FT_INT16_T
#define MPI_INT32_T FT_INT32_T
#define MPI_INT64_T FT_INT64_T
#define MPI_FLOAT FT_FLOAT
#define MPI_DOUBLE FT_DOUBLE
#define MPI_C_BOOL FT_C_BOOL
#define MPI_LONG_LONG_INT FT_LONG_LONG_INT
#define MPI_LONG_LONG FT_LONG_LONG
#define MPI_SUM FT_OP_SUM
#define MPI_BAND FT_OP_BAND
#define MPI_Comm_size FT_Comm_size
#define MPI_Comm_rank FT_Comm_rank
#define MPI_Type_size FT_Type_size
#define MPI_Type_get_name FT_Type_get_name
#define MPI_Allreduce MPI_Allreduce_FT
#define MPI_Barrier FT_Barrier
#endif

#endif /* FLEXTREE_MPI_H_ */
