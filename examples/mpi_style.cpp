// A program written against the MPI spelling of the all-reduce, built against FlexTree instead
// of an MPI library: the same call the reference intercepts by shadowing MPI_Allreduce
// (allreduce_over_mpi/mpi_mod.hpp:1723-1727).  Ranks are threads of this process here; with a GPU
// communicator (ft_mpi_from_comm) the identical call reduces device buffers over NVLink.
//
//   g++ -std=c++17 -I allreduce_over_mpi_b200/csrc examples/mpi_style.cpp \
//       -L allreduce_over_mpi_b200/lib -lflextree -Wl,-rpath,$PWD/allreduce_over_mpi_b200/lib -lpthread -o mpi_style
//   FT_TOPO=2,3 FT_LONELY=1 ./mpi_style 7
#define FLEXTREE_MPI_NAMES
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>

#include "api/flextree_mpi.h"

int main(int argc, char** argv) {
  const int world = argc > 1 ? atoi(argv[1]) : 6;
  const int count = 1 << 16;
  ft_cpu_world* w = ft_cpu_world_create(world, 30.0);
  std::vector<int> rc(world, 0);
  std::vector<std::vector<float>> data(world, std::vector<float>(count));
  std::vector<std::thread> ranks;
  for (int r = 0; r < world; ++r)
    ranks.emplace_back([&, r] {
      MPI_Comm comm = ft_mpi_thread_rank(w, r);
      int size = 0, rank = -1;
      MPI_Comm_size(comm, &size);
      MPI_Comm_rank(comm, &rank);
      for (int i = 0; i < count; ++i) data[r][i] = (float)(rank + 1);
      rc[r] = MPI_Allreduce(MPI_IN_PLACE, data[r].data(), count, MPI_FLOAT, MPI_SUM, comm);
      ft_mpi_comm_free(comm);
    });
  for (auto& t : ranks) t.join();
  const float want = world * (world + 1) / 2.0f;
  int bad = 0;
  for (int r = 0; r < world; ++r) bad += rc[r] != 0 || data[r][0] != want || data[r][count - 1] != want;
  std::printf("%d ranks, every element = %g (expected %g): %s\n", world, data[0][0], want, bad ? "FAILED" : "ok");
  ft_cpu_world_destroy(w);
  return bad ? 1 : 0;
}
