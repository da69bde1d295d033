# Developer tasks (the counterparts of the reference's pixi tasks build-cli / bench / format / test-normalization / check).
PYTHON ?= python

.PHONY: build test test-gpu check ptxas format bench

build:            ## compile every CUDA source for sm_100a in-tree (and the bounds-checked debug twin)
	$(PYTHON) setup.py build_ext --inplace

test:             ## everything that needs no GPU
	$(PYTHON) -m pytest tests -q -m "not gpu"

test-gpu:         ## on a B200 (multi-GPU tests need two or more visible GPUs)
	$(PYTHON) -m pytest tests -q -m gpu

check:            ## code-generation checks: required and forbidden instructions in the sources, bounded waits, ptxas table
	$(PYTHON) -m pytest tests/test_sources.py tests/test_launcher_validation.py -q
	$(PYTHON) -m scalingcontrasts_b200.utils.ptxas_report profiles/ptxas.md

ptxas:            ## registers, spills and shared memory of every kernel -> profiles/ptxas.md
	$(PYTHON) -m scalingcontrasts_b200.utils.ptxas_report profiles/ptxas.md

format:           ## clang-format over the native sources (only where the tool exists)
	@command -v clang-format >/dev/null && clang-format -i scalingcontrasts_b200/csrc/*.cu scalingcontrasts_b200/csrc/*.cuh \
		scalingcontrasts_b200/csrc/*.cpp scalingcontrasts_b200/csrc/*.h || echo "clang-format is not installed"

bench:            ## the headline training step on one GPU, one JSON line
	$(PYTHON) bench.py
