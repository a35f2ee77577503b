/* Shared-memory MPI subset: exactly the surface the reference's allreduce_over_mpi sources
 * use (13 functions, 11 datatype handles, 2 operators).  Ranks are separate processes of one
 * node that find each other through POSIX shared memory named after FTSHIM_SESSION (or
 * MASTER_PORT); rank and size come from RANK / WORLD_SIZE (what torch.distributed.run sets)
 * or FTSHIM_RANK / FTSHIM_SIZE.  Point-to-point messages are byte streams through one
 * single-producer single-consumer ring per ordered pair of ranks; every message in the
 * reference uses tag 0, so per-pair FIFO order is all the matching that is needed.
 * This exists only so that the unmodified reference can be built and timed on a machine
 * without an MPI installation; it is not part of the FlexTree library. */
#ifndef FTSHIM_MPI_H_
#define FTSHIM_MPI_H_
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int MPI_Comm;
typedef int MPI_Datatype;
typedef int MPI_Op;
typedef struct { int slot; } MPI_Request;
typedef struct { int MPI_SOURCE, MPI_TAG, MPI_ERROR; } MPI_Status;

#define MPI_COMM_WORLD 0
#define MPI_SUCCESS 0
#define MPI_IN_PLACE ((void*)1)
#define MPI_THREAD_MULTIPLE 3
#define MPI_STATUSES_IGNORE ((MPI_Status*)0)

#define MPI_UINT8_T 1
#define MPI_INT8_T 2
#define MPI_UINT16_T 3
#define MPI_INT16_T 4
#define MPI_INT32_T 5
#define MPI_INT64_T 6
#define MPI_FLOAT 7
#define MPI_DOUBLE 8
#define MPI_C_BOOL 9
#define MPI_LONG_LONG_INT 10
#define MPI_LONG_LONG 11

#define MPI_SUM 1
#define MPI_BAND 2

int MPI_Init_thread(int* argc, char*** argv, int required, int* provided);
int MPI_Finalize(void);
int MPI_Comm_size(MPI_Comm comm, int* size);
int MPI_Comm_rank(MPI_Comm comm, int* rank);
int MPI_Comm_split(MPI_Comm comm, int color, int key, MPI_Comm* newcomm);
int MPI_Type_size(MPI_Datatype t, int* size);
int MPI_Type_get_name(MPI_Datatype t, char* name, int* len);
int MPI_Isend(const void* buf, int count, MPI_Datatype t, int dest, int tag, MPI_Comm comm, MPI_Request* req);
int MPI_Irecv(void* buf, int count, MPI_Datatype t, int source, int tag, MPI_Comm comm, MPI_Request* req);
int MPI_Waitall(int count, MPI_Request reqs[], MPI_Status statuses[]);
int MPI_Barrier(MPI_Comm comm);
int MPI_Allreduce(const void* sendbuf, void* recvbuf, int count, MPI_Datatype t, MPI_Op op, MPI_Comm comm);
double MPI_Wtime(void);

#ifdef __cplusplus
}
#endif
#endif
