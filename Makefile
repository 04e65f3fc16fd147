# Convenience targets (the role of the reference's SConstruct + apps/helloworld/Makefile): the shared library with the
# C++ runtime and the sm_100a kernels, the C++ demo, the test suites.
PYTHON ?= python

.PHONY: lib helloworld test test-gpu bench clean

lib:
	$(PYTHON) -c "import __graft_entry__ as g; g.build()"

helloworld: lib
	$(MAKE) -C apps/helloworld

test: lib
	$(PYTHON) -m pytest tests -q -m "not gpu"

test-gpu: lib
	$(PYTHON) -m pytest tests -q -m gpu

bench: lib
	$(PYTHON) bench.py

clean:
	$(MAKE) -C apps/helloworld clean
	$(MAKE) -C tests/native clean
	rm -rf build/native
	rm -f geeps_b200/lib/libgeeps_b200.so geeps_b200/lib/libgeeps_b200.so.hash
