# Convenience targets (reference: Makefile). Everything is built in-tree; nothing here kills processes by pattern.
PY ?= python

.PHONY: build force test test-gpu bench smoke clean

build:
	$(PY) -m disagmoe_b200.build

force:
	$(PY) -m disagmoe_b200.build --force

test: build
	$(PY) -m pytest tests -x -q -m "not gpu"

test-gpu: build
	$(PY) -m pytest tests -x -q -m gpu

smoke: build
	$(PY) __graft_entry__.py

bench: build
	$(PY) bench.py --gpus 1 --steps 20 --warmup 3

clean:
	rm -rf disagmoe_b200/lib disagmoe_b200/_variants disagmoe_b200/build
	rm -f disagmoe_b200/disagmoe_c*.so
