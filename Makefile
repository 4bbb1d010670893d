# Common entry points. GPU targets expect a B200 (sm_100a).
PY ?= python
NPROC ?= 8

.PHONY: build test-cpu test-gpu test-multigpu bench bench-multi bench-band verify-records kernel-bench train clean

build:            ## compile halo_b200/lib/libhalo_b200.so for sm_100a
	$(PY) -c "import __graft_entry__ as g; g.build()"

test-cpu:         ## everything that runs without a GPU (gloo ranks for the multi-process paths)
	$(PY) -m pytest tests -q -m "not gpu"

test-gpu: build   ## kernel numerics and model tests on one GPU
	$(PY) -m pytest tests -q -m gpu

test-multigpu: build   ## peer-memory paths on two GPUs
	$(PY) -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 tests/multigpu/check_ranks.py

bench: build      ## flagship benchmark on one GPU
	$(PY) bench.py

bench-multi: build
	$(PY) -m torch.distributed.run --nnodes=1 --nproc-per-node $(NPROC) --master-addr 127.0.0.1 bench.py --gpus $(NPROC)

bench-band: build   ## hold the one-GPU benchmark to its stored band (BAND=<name> picks another; see benchmarks/band.py --list)
	$(PY) bench.py --steps 3 --warmup 3 | $(PY) benchmarks/band.py $(or $(BAND),moe30b_ep1_n1)

verify-records:   ## numerics unchanged by a change: make verify-records BASE=<records.json written at the base commit>
	$(PY) benchmarks/records.py record /tmp/halo_b200_head_records.json
	$(PY) benchmarks/records.py compare $(BASE) /tmp/halo_b200_head_records.json

kernel-bench: build
	$(PY) benchmarks/kernels.py

train:            ## make train METHOD=sft CONFIG=examples/sft_tiny_moe.yaml NPROC=1
	$(PY) -m halo_b200.cli launch $(METHOD) $(CONFIG) -n $(NPROC)

clean:
	rm -f halo_b200/lib/libhalo_b200.so halo_b200/lib/*.o
