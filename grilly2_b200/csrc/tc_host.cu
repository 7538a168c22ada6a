// Host side of the tensor-map helpers: cuTensorMapEncodeTiled is reached
// through the runtime's driver entry point lookup, so the library does not
// link against libcuda (and still loads on a machine without a driver).
#include "gq_internal.h"
#include "tc_common.cuh"

namespace gq {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
        if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !p)
            fail("cuTensorMapEncodeTiled is not available from this driver (%s)", cudaGetErrorString(e));
        fn = reinterpret_cast<EncodeFn>(p);
    }
    return fn;
}

CUtensorMap make_tensor_map_2d(const void* base, CUtensorMapDataType type, uint32_t elem_bytes, uint64_t cols, uint64_t rows,
                               uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows, Swizzle swizzle) {
    if (reinterpret_cast<uintptr_t>(base) & 15) fail("tensor map: the base address must be 16-byte aligned");
    if (pitch_bytes & 15) fail("tensor map: the row pitch (%llu bytes) must be a multiple of 16", (unsigned long long)pitch_bytes);
    if ((uint64_t)box_cols * elem_bytes & 15) fail("tensor map: the box's inner extent must be a multiple of 16 bytes");
    CUtensorMap map;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUtensorMapSwizzle sw = swizzle == Swizzle::B128  ? CU_TENSOR_MAP_SWIZZLE_128B
                                  : swizzle == Swizzle::B64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                  : swizzle == Swizzle::B32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                                            : CU_TENSOR_MAP_SWIZZLE_NONE;
    CUresult r = encode_fn()(&map, type, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) fail("cuTensorMapEncodeTiled failed with code %d (cols %llu, rows %llu, pitch %llu, box %u x %u)", (int)r,
                                (unsigned long long)cols, (unsigned long long)rows, (unsigned long long)pitch_bytes, box_cols, box_rows);
    return map;
}

}  // namespace gq
