// Tensor-map (TMA descriptor) encoding for the convolution launchers. The one driver call is
// reached through cudaGetDriverEntryPoint, so the library has no link-time dependency on libcuda.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>

#include "tc_ptx.cuh"

namespace xb200 {

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
                cudaSuccess || q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

// The last few encodings are kept per thread: a layer is launched over and over with the same
// buffers, and for one-image batches the driver calls were a visible part of the launch.
struct Key {
    const void *ptr;
    uint64_t dim[4], stride[3];
    uint32_t box[4], rank;
};

bool encode_cached(CUtensorMap *map, const Key &k) {
    struct Entry {
        Key key;
        CUtensorMap map;
        bool used;
    };
    constexpr int kEntries = 12;
    thread_local Entry cache[kEntries] = {};
    thread_local int next = 0;
    for (int i = 0; i < kEntries; i++)
        if (cache[i].used && !memcmp(&cache[i].key, &k, sizeof(Key))) {
            *map = cache[i].map;
            return true;
        }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUtensorMapSwizzle sw = k.box[0] == 128  ? CU_TENSOR_MAP_SWIZZLE_128B
                                  : k.box[0] == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                   : CU_TENSOR_MAP_SWIZZLE_32B;
    if (fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, k.rank, const_cast<void *>(k.ptr), k.dim, k.stride,
           k.box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    Entry &slot = cache[next];
    next = (next + 1) % kEntries;
    slot.key = k;
    slot.map = *map;
    slot.used = true;
    return true;
}

}  // namespace

bool encode_bytes_2d(CUtensorMap *map, const void *ptr, uint64_t rows, uint64_t row_bytes,
                     uint32_t box_bytes, uint32_t box_rows) {
    Key k;
    memset(&k, 0, sizeof k);
    k.ptr = ptr; k.rank = 2;
    k.dim[0] = row_bytes; k.dim[1] = rows;
    k.stride[0] = row_bytes;
    k.box[0] = box_bytes; k.box[1] = box_rows;
    return encode_cached(map, k);
}

bool encode_bytes_4d(CUtensorMap *map, const void *ptr, uint64_t row_bytes, uint64_t d1,
                     uint64_t d2, uint64_t d3, uint64_t s1, uint64_t s2, uint64_t s3,
                     uint32_t box_bytes, uint32_t box1, uint32_t box2) {
    Key k;
    memset(&k, 0, sizeof k);
    k.ptr = ptr; k.rank = 4;
    k.dim[0] = row_bytes; k.dim[1] = d1; k.dim[2] = d2; k.dim[3] = d3;
    k.stride[0] = s1; k.stride[1] = s2; k.stride[2] = s3;
    k.box[0] = box_bytes; k.box[1] = box1; k.box[2] = box2; k.box[3] = 1;
    return encode_cached(map, k);
}

}  // namespace xb200
