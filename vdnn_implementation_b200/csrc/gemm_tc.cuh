// tcgen05 contraction engine (placeholder until the kernel lands: reports every shape as
// unsupported so that the dispatcher uses the FFMA engine).
#pragma once

#include "gemm_operands.cuh"

namespace vdnn {
namespace tc {

template <class OpA, class OpB>
inline bool supported(int, int, int) { return false; }

template <class OpA, class OpB, bool AKC, bool BKC>
int launch(const OpA&, const OpB&, const Epilogue&, int, int, int, int, int, cudaStream_t) {
    return VDNN_ERR_UNSUPPORTED;
}

}  // namespace tc
}  // namespace vdnn
