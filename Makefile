# Common entry points.  Everything is plain Python underneath; see README.md.
PYTHON ?= python
GPUS ?= 1

.PHONY: build test test-gpu bench bench-reference doctor clean

build:            ## nvcc (sm_100a) -> rwkv7m_b200/_C.so, g++ -> rwkv7m_b200/_host.so
	$(PYTHON) -c "import __graft_entry__ as g; g.build()"

test: build       ## CPU suite: oracle, API, tools, gloo data / tensor parallel
	$(PYTHON) -m pytest tests -x -q -m "not gpu"

test-gpu: build   ## B200 suite: every kernel against the fp32 PyTorch oracle
	$(PYTHON) -m pytest tests -x -q -m gpu

bench: build      ## headline training step (1.5B, 8 x 4096 tokens per GPU); GPUS=N for N > 1
ifeq ($(GPUS),1)
	$(PYTHON) bench.py --gpus 1 --steps 4 --warmup 3
else
	$(PYTHON) -m torch.distributed.run --nnodes=1 --nproc-per-node $(GPUS) --master-addr 127.0.0.1 bench.py --gpus $(GPUS) --steps 4 --warmup 3
endif

bench-reference:  ## the reference arm (prints its "unavailable" line where the reference cannot be installed)
	$(PYTHON) bench.py --impl reference --gpus 1 --steps 4 --warmup 3

doctor:           ## what this installation can run
	$(PYTHON) -m rwkv7m_b200.cli.doctor

clean:
	rm -rf rwkv7m_b200/build rwkv7m_b200/_C.so rwkv7m_b200/_host.so
