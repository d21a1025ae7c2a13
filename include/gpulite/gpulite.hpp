// Stand-in for the header of the same name that the reference's JAX binding includes
// (sphericart-jax/src/sphericart_jax_cuda.cpp:15) and whose GPULITE_CUDART_CALL it wraps around
// cudaPointerGetAttributes (:83, :127, :177).
//
// The reference reaches the CUDA runtime through gpulite because it loads the runtime with dlopen
// and compiles its kernels at run time. This library links the CUDA runtime directly and ships
// kernels compiled ahead of time for sm_100a, so all that a binding built against it needs from
// <gpulite/gpulite.hpp> is (a) the CUDA runtime's types and functions under their usual names and
// (b) the checking macro. Put this directory's parent on the include path in place of gpulite's
// and sphericart_jax_cuda.cpp compiles unchanged against libsphericart_b200.
#ifndef SPHERICART_B200_GPULITE_SHIM_HPP
#define SPHERICART_B200_GPULITE_SHIM_HPP

#include <cuda_runtime_api.h>

#include <sstream>
#include <stdexcept>

namespace gpulite_shim {

inline void check_cudart(cudaError_t status, const char* expression, const char* file, int line) {
    if (status == cudaSuccess) return;
    std::ostringstream message;
    message << "CUDA runtime call failed: " << expression << " -> " << cudaGetErrorName(status) << " ("
            << cudaGetErrorString(status) << ") at " << file << ":" << line;
    throw std::runtime_error(message.str());
}

}  // namespace gpulite_shim

// Evaluates a CUDA runtime call and throws std::runtime_error if it did not return cudaSuccess.
#define GPULITE_CUDART_CALL(call) ::gpulite_shim::check_cudart((call), #call, __FILE__, __LINE__)

#endif
