# Developer entry points (reference: moe-engine/Makefile).
PY ?= python

.PHONY: help build test-cpu test-gpu test-multigpu smoke bench benchmark benchmark-gpu bench-kernels validate validate-config reproduce chaos chaos-a chaos-b lint clean

help:             ## list the targets
	@grep -E '^[a-z-]+: .*##' Makefile | sed -E 's/:.*## / - /'

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

benchmark:        ## router / MoE-layer / conservation micro-benchmarks on CPU
	$(PY) benchmarks/run_benchmark.py

benchmark-gpu:    ## the same on one B200 (bf16)
	$(PY) benchmarks/run_benchmark.py --cuda --skip-cpu

bench-kernels:    ## every kernel case against the measured HBM / cuBLAS peaks
	for c in router gemm_dense grouped_fwd1 grouped_fwd2 grouped_dgrad grouped_wgrad adamw rmsnorm gather combine; do \
	  $(PY) benchmarks/kernel_cases.py $$c; done

validate-config: validate

validate:         ## every shipped YAML config
	$(PY) scripts/validate_config.py configs

chaos: chaos-b chaos-a  ## both failure scenarios (gloo ranks on CPU, host-side fault injection only)

chaos-b:          ## storage stall: training continues while a checkpoint write hangs
	GLOO_SOCKET_IFNAME=lo $(PY) -m pytest tests/test_chaos.py -q -k "stall or scenario_b"

chaos-a:          ## a rank is killed and the job restarts from the newest checkpoint every rank has
	GLOO_SOCKET_IFNAME=lo $(PY) -m pytest tests/test_chaos.py -q -k "kill or restart or scenario_a"

lint:             ## byte-compile every source (ruff / mypy when installed)
	$(PY) -m compileall -q composed_mixture_of_experts_engine_b200 pkg scripts benchmarks tests train.py bench.py
	-ruff check composed_mixture_of_experts_engine_b200 train.py bench.py benchmarks scripts

reproduce:        ## the numbers of the benchmark tables, one command
	$(PY) scripts/reproduce.py

clean:            ## built objects and caches
	rm -rf composed_mixture_of_experts_engine_b200/_build .pytest_cache
