# Shared build rules of the tutorials: plain nvcc against the headers and the shared library of the package.
#   make PKG=<path to the mscclpp_b200 package directory>     (default: the one inside this repository)
PKG ?= $(abspath $(dir $(lastword $(MAKEFILE_LIST)))/../../mscclpp_b200)
NVCC ?= nvcc
NVCCFLAGS ?= -std=c++17 -O2 -lineinfo -gencode arch=compute_100a,code=sm_100a
INCLUDES = -I$(PKG)/csrc/include
LDFLAGS = -L$(PKG)/lib -lmscclpp_b200 -Xlinker -rpath -Xlinker $(PKG)/lib

%: %.cu
	$(NVCC) $(NVCCFLAGS) $(INCLUDES) $< -o $@ $(LDFLAGS)
