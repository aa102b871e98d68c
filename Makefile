# nanoplm-b200: build, test and benchmark targets.
# The kernels are compiled in-tree for sm_100a with nvcc (no GPU needed to build).

PYTHON ?= python
NPROC  ?= 8

.PHONY: help build test test-fast test-gpu test-multigpu parity bench bench-reference bench-multi \
        bench-kernels bench-data clean

help:
	@echo "build            compile every CUDA / C++ extension into nanoplm_b200/_lib"
	@echo "test             CPU tests (contracts, pipelines, gloo ranks, recovery, reference parity)"
	@echo "test-fast        the same, in parallel (pytest-xdist)"
	@echo "test-gpu         kernel and model tests on one B200"
	@echo "test-multigpu    engines, MoE, Muon, time-outs on >= 2 GPUs"
	@echo "parity           only the tests against the reference package / its own test files"
	@echo "bench            flagship training step on one GPU (one JSON line)"
	@echo "bench-reference  the unmodified reference on the same config"
	@echo "bench-multi      the same on NPROC GPUs (default 8)"
	@echo "bench-kernels    kernel micro-benchmarks; bench-data: host data pipeline (no GPU)"

build:
	$(PYTHON) -m nanoplm_b200.csrc.build

test:
	$(PYTHON) -m pytest tests -q -m "not gpu"

test-fast:
	$(PYTHON) -m pytest tests -q -m "not gpu" -n auto

test-gpu:
	$(PYTHON) -m pytest tests -q -m gpu

test-multigpu:
	$(PYTHON) -m pytest tests/test_multigpu.py -q

parity:
	$(PYTHON) -m pytest tests/test_reference_parity.py tests/test_reference_own_tests.py tests/test_teacher_hf_parity.py -q

bench:
	$(PYTHON) bench.py --gpus 1 --steps 3 --warmup 3

bench-reference:
	$(PYTHON) bench.py --impl reference --gpus 1 --steps 3 --warmup 3

bench-multi:
	$(PYTHON) -m torch.distributed.run --nnodes=1 --nproc-per-node $(NPROC) --master-addr 127.0.0.1 \
	    --master-port 29511 bench.py --gpus $(NPROC) --steps 3 --warmup 3

bench-kernels:
	$(PYTHON) -m nanoplm_b200.bench.kernel_bench

bench-data:
	$(PYTHON) -m nanoplm_b200.bench.data_bench --sequences 12000

clean:
	$(PYTHON) -c "import pathlib, shutil; [shutil.rmtree(p, ignore_errors=True) for p in pathlib.Path('.').rglob('__pycache__')]; shutil.rmtree('.pytest_cache', ignore_errors=True)"
