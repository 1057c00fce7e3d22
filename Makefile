# Build of libdccl.so, the command-line tools and the examples.
#
#   make                 library + tools for B200 (sm_100a), CUDA enabled
#   make CUDA=0          host-only library (no nvcc needed; device calls are refused)
#   make SANITIZE=address|thread|undefined CXX=/usr/bin/g++ CC=/usr/bin/gcc   instrument the host code (host-only build;
#                        a compiler wrapper that links statically may lack the sanitizer runtimes)
#   make BOUNDS=1        debug build of the device code in build-bounds/: every kernel checks the pool ranges it is
#                        about to use and reports DEV_BOUNDS instead of touching memory outside them
#   make SIM=1 lib       host simulation of the non-multimem kernels in build-sim/: the kernel sources compiled as C++,
#                        every CUDA thread an OS thread; the single-GPU emulation tests then run without a GPU
#                        (DCCL_LIBRARY=build-sim/libdccl.so, see tests/test_kernel_sim.py)
#   make install PREFIX=/opt/dccl         headers, library, tools, CMake package file
#
# Everything lands in build/; the shared library is also copied into the Python
# package (dccl_b200/lib/) so that it is found next to the bindings.

CUDA ?= 1
CUDA_HOME ?= /usr/local/cuda
NVCC ?= $(CUDA_HOME)/bin/nvcc
CXX ?= g++
BUILD ?= build
CACHELINE := $(shell getconf LEVEL1_DCACHE_LINESIZE 2>/dev/null || echo 64)
ifeq ($(CACHELINE),0)
CACHELINE := 64
endif
ifeq ($(CACHELINE),)
CACHELINE := 64
endif

CXXFLAGS := -std=c++17 -O3 -fPIC -Wall -Wextra -Wno-unused-parameter -Iinclude -DCACHELINE_SIZE=$(CACHELINE) -DENABLE_EVALUATION=1 -pthread
LDFLAGS := -pthread -lrt -ldl
NVCCFLAGS := -std=c++17 -O3 -lineinfo -gencode arch=compute_100a,code=sm_100a -Xcompiler -fPIC -Iinclude \
             -DCACHELINE_SIZE=$(CACHELINE) -DENABLE_EVALUATION=1 -DDCCL_WITH_CUDA_RUNTIME
ifdef PTXAS_V
NVCCFLAGS += -Xptxas -v
endif
ifdef BOUNDS
NVCCFLAGS += -DDCCL_DEBUG_BOUNDS
BUILD := build-bounds
endif
ifdef SIM
CUDA := 0
BUILD := build-sim
endif
ifdef SANITIZE
CUDA := 0
CXXFLAGS += -fsanitize=$(SANITIZE) -fno-omit-frame-pointer -g
LDFLAGS += -fsanitize=$(SANITIZE)
BUILD := build-$(SANITIZE)
endif

HOST_SRCS := csrc/core/config.cpp csrc/core/log.cpp csrc/core/timestamp.cpp \
             csrc/bootstrap/bootstrap.cpp csrc/cpu/cpu_backend.cpp \
             csrc/api/dccl_api.cpp csrc/api/composed.cpp csrc/api/c_api.cpp csrc/api/names.cpp csrc/tuner/tuner.cpp
ifeq ($(CUDA),1)
CU_SRCS := $(wildcard csrc/gpu/*.cu) $(wildcard csrc/kernels/*.cu)
CXXFLAGS += -DDCCL_WITH_CUDA -DDCCL_WITH_CUDA_RUNTIME -I$(CUDA_HOME)/include
CUDA_LIBS := -L$(CUDA_HOME)/lib64 -lcudart_static
TOOL_DEFS := -DDCCL_WITH_CUDA
else
HOST_SRCS += csrc/gpu/gpu_stub.cpp
CU_SRCS :=
CUDA_LIBS :=
TOOL_DEFS :=
endif

ifdef SIM
HOST_SRCS += csrc/sim/sim_runtime.cpp
CU_SRCS := csrc/gpu/emu.cu csrc/gpu/canary.cu csrc/kernels/twoshot.cu csrc/kernels/ring.cu csrc/kernels/hd.cu csrc/kernels/direct.cu \
           csrc/kernels/oneshot_ll.cu csrc/kernels/ll_collectives.cu csrc/kernels/ll_twoshot.cu csrc/kernels/p2p.cu \
           csrc/kernels/nvls.cu csrc/kernels/nvls_pipe.cu csrc/kernels/nvls_rooted.cu
# -O2 and no strict aliasing: the kernels reinterpret 16-byte vectors the way device code does
SIM_FLAGS := -Icsrc/sim/include -DDCCL_HOST_SIM -fno-strict-aliasing -Wno-attributes -Wno-unknown-pragmas -Wno-maybe-uninitialized
ifdef BOUNDS
SIM_FLAGS += -DDCCL_DEBUG_BOUNDS
BUILD := build-sim-bounds
endif
endif
HOST_OBJS := $(patsubst %.cpp,$(BUILD)/obj/%.o,$(HOST_SRCS))
CU_OBJS := $(patsubst %.cu,$(BUILD)/obj/%.cu.o,$(CU_SRCS))
LIB := $(BUILD)/libdccl.so
TOOLS := $(BUILD)/dccl_cli $(BUILD)/p2p_perf $(BUILD)/helloworld $(BUILD)/nccl_names $(BUILD)/c_api_example
ifeq ($(CUDA),1)
TOOLS += $(BUILD)/nccl_cli $(BUILD)/dccl_sweep $(BUILD)/dccl_topo
endif

.PHONY: all lib tools clean install
PREFIX ?= /usr/local
all: lib tools
# only the default build directory feeds the Python package: an instrumented library must not replace the real one
ifeq ($(BUILD),build)
lib: $(LIB) dccl_b200/lib/libdccl.so
else
lib: $(LIB)
endif
tools: $(TOOLS)

$(BUILD)/obj/%.o: %.cpp $(wildcard include/dccl/*.hpp) $(wildcard csrc/*/*.hpp)
	@mkdir -p $(dir $@)
	$(CXX) $(CXXFLAGS) $(SIM_FLAGS) -c $< -o $@

ifdef SIM
$(BUILD)/obj/%.cu.o: %.cu $(wildcard include/dccl/*.hpp) $(wildcard csrc/*/*.hpp) $(wildcard csrc/*/*.cuh) $(wildcard csrc/sim/include/*.h)
	@mkdir -p $(dir $@)
	$(CXX) -x c++ $(filter-out -O3,$(CXXFLAGS)) -O2 $(SIM_FLAGS) -c $< -o $@
else
$(BUILD)/obj/%.cu.o: %.cu $(wildcard include/dccl/*.hpp) $(wildcard csrc/*/*.hpp) $(wildcard csrc/*/*.cuh)
	@mkdir -p $(dir $@)
	$(NVCC) $(NVCCFLAGS) -c $< -o $@
endif

$(LIB): $(HOST_OBJS) $(CU_OBJS)
	$(CXX) -shared -o $@ $^ $(CUDA_LIBS) $(LDFLAGS) -Wl,--exclude-libs,ALL -Wl,-Bsymbolic

dccl_b200/lib/libdccl.so: $(LIB)
	@mkdir -p dccl_b200/lib
	cp $(LIB) $@

$(BUILD)/dccl_cli: tools/dccl_cli.cpp tools/tool_common.hpp $(LIB)
	$(CXX) $(CXXFLAGS) $(TOOL_DEFS) $< -o $@ -L$(BUILD) -ldccl -Wl,-rpath,'$$ORIGIN' $(CUDA_LIBS) $(LDFLAGS)

$(BUILD)/p2p_perf: tools/p2p_perf.cpp tools/tool_common.hpp $(LIB)
	$(CXX) $(CXXFLAGS) $(TOOL_DEFS) $< -o $@ -L$(BUILD) -ldccl -Wl,-rpath,'$$ORIGIN' $(CUDA_LIBS) $(LDFLAGS)

$(BUILD)/helloworld: examples/helloworld/main.cpp $(LIB)
	$(CXX) $(CXXFLAGS) $< -o $@ -L$(BUILD) -ldccl -Wl,-rpath,'$$ORIGIN' $(LDFLAGS)

$(BUILD)/nccl_names: examples/nccl_names/main.cpp $(LIB)
	$(CXX) $(CXXFLAGS) $< -o $@ -L$(BUILD) -ldccl -Wl,-rpath,'$$ORIGIN' $(LDFLAGS)

$(BUILD)/c_api_example: examples/c_api/main.c include/dccl/dccl_c.h $(LIB)
	$(CC) -O2 -Wall -Iinclude $< -o $@ -L$(BUILD) -ldccl -Wl,-rpath,'$$ORIGIN' $(LDFLAGS)

# comparator: the same workload through stock NCCL (found at run time with dlopen)
$(BUILD)/nccl_cli: tools/nccl_cli.cpp tools/tool_common.hpp $(LIB)
	$(CXX) $(CXXFLAGS) $(TOOL_DEFS) $< -o $@ -L$(BUILD) -ldccl -Wl,-rpath,'$$ORIGIN' $(CUDA_LIBS) $(LDFLAGS)

$(BUILD)/dccl_topo: tools/dccl_topo.cpp $(LIB)
	$(CXX) $(CXXFLAGS) $(TOOL_DEFS) $< -o $@ -L$(BUILD) -ldccl -Wl,-rpath,'$$ORIGIN' $(CUDA_LIBS) $(LDFLAGS)

$(BUILD)/dccl_sweep: tools/dccl_sweep.cpp tools/tool_common.hpp $(LIB)
	$(CXX) $(CXXFLAGS) $(TOOL_DEFS) $< -o $@ -L$(BUILD) -ldccl -Wl,-rpath,'$$ORIGIN' $(CUDA_LIBS) $(LDFLAGS)

# headers, library, tools and a CMake package file (find_package(dccl))
install: all
	install -d $(PREFIX)/include/dccl $(PREFIX)/lib $(PREFIX)/bin $(PREFIX)/lib/cmake/dccl
	install -m 644 include/dccl/dccl.hpp include/dccl/dccl_c.h include/dccl/config.h $(PREFIX)/include/dccl/
	install -m 755 $(LIB) $(PREFIX)/lib/
	install -m 755 $(TOOLS) $(PREFIX)/bin/
	sed 's/@CACHELINE@/$(CACHELINE)/' dcclConfig.cmake.in > $(PREFIX)/lib/cmake/dccl/dcclConfig.cmake

clean:
	rm -rf build build-address build-thread build-undefined dccl_b200/lib
