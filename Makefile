# Thin wrapper for people who type `make`: the real build description is tileccl_b200/_build.py
# (nvcc, -gencode arch=compute_100a,code=sm_100a, everything in-tree).
PYTHON ?= python

all:
	$(PYTHON) -m tileccl_b200._build

ptxas:            # registers / spills / shared memory of every kernel
	$(PYTHON) -m tileccl_b200._build --ptxas

test:
	$(PYTHON) -m pytest tests -q -m "not gpu"

test-gpu:
	$(PYTHON) -m pytest tests -q -m gpu

quick:            # whole suite, short presets, into reports/
	$(PYTHON) -m tileccl_b200.bench.run_all --quick

clean:
	rm -rf tileccl_b200/build tileccl_b200/bin tileccl_b200/lib/*.so

.PHONY: all ptxas test test-gpu quick clean
