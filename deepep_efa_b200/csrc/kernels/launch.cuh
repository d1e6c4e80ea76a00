// Launch helper for kernels that take one argument block per (emulated) rank.
//
// gridDim.y selects the rank. With one rank the launch is an ordinary one; with several emulated
// ranks it is cooperative, so the runtime refuses it (instead of letting it deadlock) when the whole
// grid cannot be co-resident.
#pragma once

#include <cuda_runtime.h>

#include "prims.cuh"

namespace dx {

template <typename Args, int V>
struct ArgPack {
    Args a[V];
};

template <typename Args, int V>
cudaError_t launch_ranked(void (*kernel)(const ArgPack<Args, V>), const Args* args, int num_virtual, int ctas_per_rank,
                          int threads, size_t smem, cudaStream_t stream, bool programmatic = false) {
    ArgPack<Args, V> pack;
    for (int i = 0; i < num_virtual; ++i) pack.a[i] = args[i];
    for (int i = num_virtual; i < V; ++i) pack.a[i] = args[0];
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas_per_rank, num_virtual, 1);
    cfg.blockDim = dim3(threads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (num_virtual > 1) {
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
    } else {
        // Programmatic dependent launch: the launch work of this kernel overlaps the tail of the previous kernel in
        // the stream; the kernel itself calls griddepcontrol.wait before it touches anything the predecessor wrote.
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = programmatic ? 1 : 0;
    }
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, pack);
}

// Picks the 1-rank or the 8-rank instantiation.
#define DX_LAUNCH_RANKED(KERNEL, ARGS_T, args, nv, ctas, threads, smem, stream)                                 \
    ((nv) == 1 ? ::dx::launch_ranked<ARGS_T, 1>(KERNEL<1>, args, 1, ctas, threads, smem, stream)                \
               : ::dx::launch_ranked<ARGS_T, ::dx::kMaxVirtualRanks>(KERNEL<::dx::kMaxVirtualRanks>, args, nv, \
                                                                    ctas, threads, smem, stream))

// Same, with programmatic dependent launch enabled for the single-rank instantiation.
#define DX_LAUNCH_RANKED_PDL(KERNEL, ARGS_T, args, nv, ctas, threads, smem, stream)                             \
    ((nv) == 1 ? ::dx::launch_ranked<ARGS_T, 1>(KERNEL<1>, args, 1, ctas, threads, smem, stream, true)          \
               : ::dx::launch_ranked<ARGS_T, ::dx::kMaxVirtualRanks>(KERNEL<::dx::kMaxVirtualRanks>, args, nv, \
                                                                    ctas, threads, smem, stream))

}  // namespace dx
