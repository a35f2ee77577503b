// The same MPI-spelled program as mpi_style.cpp, but started the way an MPI job is: one PROCESS per rank.
// There is no MPI library underneath: the ranks meet through a shared-memory session and pull blocks out of
// each other's buffers with process_vm_readv.  Rank, size and session come from the launcher's environment
// (FT_RANK / FT_WORLD / FT_SESSION, or RANK / WORLD_SIZE / MASTER_PORT as torch.distributed.run sets them):
//
//   g++ -std=c++17 -I allreduce_over_mpi_b200/csrc examples/mpi_style_procs.cpp \
//       -L allreduce_over_mpi_b200/lib -lflextree -Wl,-rpath,$PWD/allreduce_over_mpi_b200/lib -lpthread -o mpi_style_procs
//   for r in 0 1 2 3 4 5 6; do FT_RANK=$r FT_WORLD=7 FT_SESSION=demo FT_TOPO=2,3 FT_LONELY=1 ./mpi_style_procs & done; wait
#define FLEXTREE_MPI_NAMES
#include <cstdio>
#include <vector>

#include "api/flextree_mpi.h"

int main() {
  MPI_Comm comm = ft_mpi_proc_init_env(30.0);          // MPI_Init + MPI_COMM_WORLD
  if (!comm) { std::fprintf(stderr, "%s\n", ft_mpi_last_error()); return 2; }
  int size = 0, rank = -1;
  MPI_Comm_size(comm, &size);
  MPI_Comm_rank(comm, &rank);
  const int count = 100003;
  std::vector<double> data(count, (double)(rank + 1));
  MPI_Barrier(comm);
  const int rc = MPI_Allreduce(MPI_IN_PLACE, data.data(), count, MPI_DOUBLE, MPI_SUM, comm);
  const double want = size * (size + 1) / 2.0;
  bool ok = rc == 0 && data[0] == want && data[count - 1] == want;
  // The same call on a buffer from the world's symmetric heap is reduced in place through shared mappings
  // (no copy, no system call) - the host twin of a tensor in the GPU communicator's symmetric heap.
  ft_proc_world* world = ft_mpi_proc_world(comm);
  if (ft_proc_heap_create(world, 4 << 20) == 0) {
    double* shared = (double*)ft_proc_alloc(world, count * sizeof(double));
    for (int i = 0; i < count; ++i) shared[i] = (double)(rank + 1);
    ok = ok && MPI_Allreduce(MPI_IN_PLACE, shared, count, MPI_DOUBLE, MPI_SUM, comm) == 0 && shared[0] == want && shared[count - 1] == want;
  } else {
    ok = false;
  }
  std::printf("rank %d of %d: every element = %g (expected %g): %s\n", rank, size, data[0], want, ok ? "ok" : "FAILED");
  ft_mpi_proc_finalize(comm);                           // MPI_Finalize
  return ok ? 0 : 1;
}
