// Launch API of the grouped expert GEMM kernels (tcgen05 / TMEM / TMA, sm_100a). No torch headers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace dx {
}  // namespace dx
