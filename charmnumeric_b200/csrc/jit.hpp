// Run-time compilation of generated group kernels (NVRTC -> cubin for sm_100a) and the
// function cache keyed by the group's structural key.
//
// Counterpart of ArrayDAGGroup::compile_node / module_cache in the reference
// (src/dag_group_compile.cpp:6-56) and of MLIRJitCompiler::generateNVIDIA / loadNVIDIA
// (src/jit.cpp:463-540), which emit PTX for sm_70 and load it with the driver API.
#pragma once
#include <map>
#include <cstdint>
#include <string>
#include <vector>

#include "group_ir.hpp"

namespace cn {

struct TileConfig {
    int block = 256;  // threads per block
    int tx = 256;  // threads along the last dimension
    int r = 2;     // consecutive rows per thread
    // element strides of the arrays a stencil kernel is specialised for (0: read at run time);
    // as compile-time constants they turn every stencil arm into an immediate address offset
    long long s0 = 0, s1 = 0;
    // test hook of the staged kernels: issue no tile copies and give up waiting quickly
    bool drop_copies = false;
    int ns = 0;  // ring depth of the staged kernels (0: the generator's default)
    // flat kernels: 0 loads where they are used; 1 the next tile's inputs are requested before
    // this tile's arithmetic starts (register double buffering); 2 all loads of a tile are
    // issued up front, ahead of its arithmetic
    int prefetch = 0;
    // stencil kernels: single neighbours along the last dimension come from the neighbour
    // lanes' registers (warp shuffle) instead of their own loads
    bool shfl = false;
    // kernels of a multi-rank context can store their slab's edge rows into the neighbours'
    // mailboxes themselves (the launch arguments say when)
    bool push = false;
    // the kernel releases the next kernel of the stream as soon as all its own blocks have
    // started (instead of when they have exited).  Measured harmful: the next kernel's blocks
    // take every free slot of the SMs and wait there (CG 8192^2 888 -> 1 001 us per iteration,
    // Jacobi3D 1024^3 3.08 -> 3.68 ms), so it is off
    bool trigger = false;
    int minb = 1;    // resident blocks per SM the compiler has to leave room for (register cap)
    int fill_u = 3;  // staged producers: points per thread whose loads are issued together
};

// Compile CUDA source to a cubin image for sm_100a.  Works without a GPU.
// `log` receives the NVRTC log (warnings, errors).
int nvrtc_compile(const std::string& source, const TileConfig& tile, std::vector<char>* cubin,
                  std::string* log);

// Bytes of register spills the compiler reported in an NVRTC log (0 when it reported none).
long long spill_bytes(const std::string& log);

// Digest of everything that decides a generated kernel's machine code apart from the array
// strides it is specialised on: the generated source, the device header and the tile
// configuration.  Profile labels carry it, so that a stored measurement of a kernel can be
// told from a measurement of an earlier version of that kernel.
uint32_t code_digest(const std::string& source, const TileConfig& tile);

// Texts of the headers every generated kernel includes (embedded at build time).
extern const char* const kDeviceHeaderText;
extern const char* const kExpTableText;
// Digest of the sources of the kernels built ahead of time (matvec, dot / sum, halo copies).
extern const char* const kAotSourceDigest;

}  // namespace cn
