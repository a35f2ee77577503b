# Convenience targets; every one is a thin wrapper around a command documented in README.md.
PY ?= python
NGPU ?= 8

.PHONY: build test test-gpu bench bench-multi reference cmake clean

build:            ## libflextree.so + native tools (nvcc, sm_100a)
	$(PY) -m allreduce_over_mpi_b200.build

test: build       ## CPU suite: planner, cost model, executors, MPI-compatible entry, tools, sanitizers
	$(PY) -m pytest tests -q -m "not gpu"

test-gpu: build   ## kernels on one GPU (emulated ranks) and multi-process runs on >= 2 GPUs
	$(PY) -m pytest tests -q -m gpu

bench: build      ## 1 GPU: n-way reduce GB/s
	$(PY) bench.py

bench-multi: build ## NGPU GPUs: all-reduce bus bandwidth (+ NCCL on the same buffer)
	$(PY) -m torch.distributed.run --nnodes=1 --nproc-per-node $(NGPU) --master-addr 127.0.0.1 --master-port 29500 bench.py --gpus $(NGPU)

reference:        ## build the unmodified reference for `bench.py --impl reference` and baseline/config1.py
	$(PY) baseline/install_reference.py

cmake:            ## the same library through CMake
	cmake -S allreduce_over_mpi_b200/csrc -B build-ft && cmake --build build-ft -j

clean:
	rm -rf allreduce_over_mpi_b200/csrc/build allreduce_over_mpi_b200/lib build-ft
