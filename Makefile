# Convenience targets over the Python build driver (parameter_server_b200/_build.py does the work:
# nvcc for sm_100a, g++ for the host runtime). `make` builds everything in-tree.
PY      ?= python
CXX     ?= g++
CORE    := parameter_server_b200/csrc/core
LIBDIR  := parameter_server_b200/lib
EXAMPLES := $(patsubst examples/cpp/%.cc,build/%,$(wildcard examples/cpp/*.cc))

all:                  ## CUDA library, _core module, bin/psb_linear
	$(PY) __graft_entry__.py

core:                 ## host runtime only (no nvcc needed)
	$(PY) -m parameter_server_b200._build --core

lib:                  ## lib/libpsb.a and lib/libpsbmain.a for C++ programs
	$(PY) -m parameter_server_b200._build --static

examples: lib $(EXAMPLES)   ## the C++ programs under examples/cpp, linked against the static libraries

build/%: examples/cpp/%.cc $(LIBDIR)/libpsb.a $(LIBDIR)/libpsbmain.a
	@mkdir -p build
	$(CXX) -O2 -std=c++17 -Wall -pthread -I$(CORE) $< $(if $(shell grep -l "^int main" $<),,$(LIBDIR)/libpsbmain.a) $(LIBDIR)/libpsb.a -lz -o $@

test:                 ## everything that needs no GPU
	$(PY) -m pytest tests -q -m "not gpu"

gputest:              ## kernels against fp32 references (needs a B200)
	$(PY) -m pytest tests -q -m gpu

bench:
	$(PY) bench.py

sanitize:             ## node binary under ASan+UBSan and under TSan
	$(PY) -m parameter_server_b200._build --sanitize
	$(PY) -m parameter_server_b200._build --sanitize=thread

doc:                  ## Doxygen over the C++ headers -> docs/doxygen
	cd docs && doxygen Doxyfile

clean:
	rm -rf build parameter_server_b200/csrc/build parameter_server_b200/lib parameter_server_b200/bin
	rm -f parameter_server_b200/*.so parameter_server_b200/*.stamp

.PHONY: all core lib examples test gputest bench sanitize doc clean
