// Host-side tensor-map encoding.  The driver entry point is looked up at run time so the
// library links against the CUDA runtime only.
#include <mutex>

#include "hx_tma.cuh"

namespace hx {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            cudaGetLastError();
    });
    return fn;
}

hx_status encode_tensor_map(CUtensorMap *map, int dtype, int rank, const void *base, const uint64_t *dims,
                            const uint64_t *strides_bytes, const uint32_t *box, bool swizzle128) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return fail(HX_ERR_BACKEND, "cuTensorMapEncodeTiled is not available from this driver");
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0)
        return fail(HX_ERR_UNSUPPORTED_OPERATION, "tensor base %p is not 16-byte aligned (TMA rule)", base);
    for (int i = 0; i + 1 < rank; ++i)
        if ((strides_bytes[i] & 15) != 0)
            return fail(HX_ERR_UNSUPPORTED_OPERATION, "tensor stride %llu bytes is not a multiple of 16 (TMA rule)",
                        (unsigned long long)strides_bytes[i]);
    CUtensorMapDataType dt = dtype == HX_F32   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                             : dtype == HX_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    cuuint64_t gdims[5], gstr[4];
    cuuint32_t gbox[5], estr[5];
    for (int i = 0; i < rank; ++i) {
        gdims[i] = dims[i];
        gbox[i] = box[i];
        estr[i] = 1;
        if (i + 1 < rank) gstr[i] = strides_bytes[i];
    }
    CUresult r = fn(map, dt, (cuuint32_t)rank, const_cast<void *>(base), gdims, gstr, gbox, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(HX_ERR_BACKEND, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return HX_OK;
}

}  // namespace hx
