// Minimal stand-in for CUDA's <vector_types.h>, found through -I when the
// reference's discrete_kernels.cu is compiled as host C++.
#pragma once
struct int3 { int x, y, z; };
struct int4 { int x, y, z, w; };
