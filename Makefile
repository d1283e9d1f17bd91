# Every target runs from the repository root. The GPU targets need a B200.
PY ?= python

.PHONY: build
build:            ## nvcc (sm_100a) -> ops/_lib/libpdb200.so, g++ -> ops/_lib/libpdhost.so
	$(PY) -m param_decomp_b200.ops.build

.PHONY: test
test:             ## CPU suite (gloo ranks for the multi-process paths)
	$(PY) -m pytest tests -q -m "not gpu"

.PHONY: test-gpu
test-gpu:         ## GPU suite (multi-GPU tests skip below two GPUs)
	$(PY) -m pytest tests -q -m gpu

.PHONY: smoke
smoke: build      ## one tiny fused step on cuda:0
	$(PY) __graft_entry__.py smoke

.PHONY: bench
bench:            ## headline benchmark on one GPU; N > 1: python -m torch.distributed.run ... bench.py --gpus N
	$(PY) bench.py --gpus 1 --steps 8 --warmup 3

.PHONY: invariance
invariance:       ## one process against four gloo ranks (data x tensor parallel), training and evaluation metrics
	$(PY) -m param_decomp_b200.experiments.lm.invariance_check --world 4 --tp 2 --sharding zero1 --with-eval
