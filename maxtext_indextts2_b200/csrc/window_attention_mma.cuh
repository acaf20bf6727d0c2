// Tensor-core arm of the windowed sigmoid attention (window_attention.cuh has the contract and the row kernel).
#pragma once

#include "window_attention.cuh"

namespace mtx {

template <typename T>
inline bool window_mma_usable(const WindowAttnArgs<T>&) { return false; }
inline int window_mma_min_rows() { return 1 << 30; }
template <typename T>
inline int launch_window_mma(const WindowAttnArgs<T>&, cudaStream_t) { return 0; }

}  // namespace mtx
