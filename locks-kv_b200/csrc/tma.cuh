// Tiled tensor-map copies (TMA): the device-side load and the host-side
// descriptor encoder, shared by the kernels that stage cache pages with
// cp.async.bulk.tensor.  Every map covers memory of the launching GPU only and
// no load carries a cluster-multicast qualifier.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace locks {

#ifdef __CUDACC__
// one box of a 2-D tensor map -> shared memory; x (innermost, in elements) times
// the element size must be a multiple of 16 bytes
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x,
                                            int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
#endif

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time
// dependency on the driver library)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
inline EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault,
                                    &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// A bf16 matrix of `rows` rows of `row_elems` elements, `row_pitch_elems` apart,
// cut into boxes of (box_rows x 64 elements) laid out in shared memory with the
// 128-byte swizzle.  CUDA_SUCCESS or the driver's error.
inline CUresult encode_bf16_rows_sw128(CUtensorMap* map, const void* base,
                                       uint64_t row_elems, uint64_t rows,
                                       uint64_t row_pitch_elems, uint32_t box_rows) {
    EncodeTiledFn enc = encode_tiled();
    if (enc == nullptr) return CUDA_ERROR_NOT_SUPPORTED;
    const cuuint64_t gdim[2] = {(cuuint64_t)row_elems, (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)row_pitch_elems * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim,
               gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

}  // namespace locks
