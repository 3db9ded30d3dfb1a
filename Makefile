# Developer entry points (reference: moe-engine/Makefile).
PY ?= python

.PHONY: build test-cpu test-gpu test-multigpu smoke bench bench-kernels validate reproduce clean

build:            ## compile the sm_100a extension and the checkpoint writer in-tree
	$(PY) __graft_entry__.py

test-cpu:         ## tier 0 + multi-process gloo tests (no GPU needed)
	$(PY) -m pytest tests -x -q -m "not gpu"

test-gpu:         ## kernel and module numerics on one B200
	$(PY) -m pytest tests -x -q -m "gpu and not multigpu"

test-multigpu:    ## expert-parallel / sharded-optimizer paths on >= 2 GPUs
	$(PY) -m pytest tests/test_gpu_multi.py -x -q -m gpu

smoke:            ## 5 toy steps through train.py
	$(PY) train.py --config configs/smoke.yaml --smoke --no-wandb

bench:            ## headline benchmark on one GPU
	$(PY) bench.py

bench-kernels:
	for c in router gemm_dense grouped_fwd1 grouped_fwd2 grouped_dgrad grouped_wgrad adamw rmsnorm gather combine; do \
	  $(PY) benchmarks/kernel_cases.py $$c; done

validate:
	$(PY) scripts/validate_config.py configs

reproduce:
	$(PY) scripts/reproduce.py

clean:
	rm -rf composed_mixture_of_experts_engine_b200/_build .pytest_cache
