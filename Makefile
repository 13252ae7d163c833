# Developer entry points (reference: Makefile:79-132 -- build, test, docs targets).
PY ?= python

.PHONY: build test test-gpu test-all lint docs bench clean

build:            ## compile the native sm_100a library (nvcc cross-compiles without a GPU)
	$(PY) -m jaxpp_b200.csrc.build

test: build       ## CPU tiers
	tests/run_tests.sh --cpu-only

test-gpu: build   ## single- and multi-GPU tiers
	tests/run_tests.sh --gpu-only

test-all: build
	tests/run_tests.sh

lint:
	$(PY) -m ruff check jaxpp_b200 tests examples bench.py

docs:             ## the documentation is plain Markdown: the top-level README, docs/ and the tutorial under examples/
	@ls README.md docs/*.md examples/tutorial.md

bench:            ## headline benchmark on one GPU (use torch.distributed.run for more, see bench.py)
	$(PY) bench.py --gpus 1

clean:
	rm -rf jaxpp_b200/_native
