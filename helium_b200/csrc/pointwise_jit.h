// Plan-time specialisation of a pointwise program: the PwProgram the interpreter would execute is printed as
// straight-line CUDA C (one statement per program instruction, shapes and view constants as literals), compiled
// for sm_100a with NVRTC and launched like any other kernel.  This is the route of the reference, which prints and
// compiles one kernel per pointwise subgraph (helium/src/cuda/instr/pointwise/jit.rs); the interpreter remains
// the fallback when the NVRTC library is not present, the program is outside the generator's range (reductions,
// bit-packed bool tensors) or a tensor breaks the 16-byte rule at launch.
#pragma once
#include <memory>
#include <string>

#include "pointwise_program.h"

namespace he {

struct PwJitModule;   // compiled code plus its per-device loaded image

// Prints the kernel for `c`.  Returns false (with a reason) when the program is outside the generator's range.
bool pw_jit_generate(const PwCompiled& c, std::string* source, std::string* why);

// Compiles (or finds in the process-wide cache) the kernel of `c`.  HE_ERR_UNSUPPORTED with a message when NVRTC is
// unavailable or the program is out of range; HE_ERR_CUDA when the compiler rejects the generated source.
int32_t pw_jit_compile(const PwCompiled& c, std::shared_ptr<PwJitModule>* out);

// Launches the kernel with the pointers of `P` (every identity-mapped tensor must be 16-byte aligned: the caller
// checks and falls back to the interpreter otherwise).
int32_t pw_jit_launch(PwJitModule& m, const PwProgram& P, int sm_count, cudaStream_t stream);

// The reduction kernel of a program with reductions (same thread-to-element mapping and combine order as the
// interpreter's pw_reduce_kernel, so both give the same bits); `grid` as computed for that kernel.
int32_t pw_jit_launch_reduce(PwJitModule& m, const PwProgram& P, const PwReduceLaunch& L, unsigned grid, cudaStream_t stream);

// true when every tensor the kernel reads or writes with 16-byte accesses is aligned for them
bool pw_jit_pointers_ok(const PwCompiled& c, const PwProgram& P);

}  // namespace he
