// Cached TMA tensor maps (cuTensorMapEncodeTiled through the runtime's driver entry point) for the tensor-core kernels.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "tsp_common.cuh"

namespace tsp {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

// Cached tensor map over bytes (rank <= 5). Weights are immutable imports and scratch buffers are reused, so a map
// depends only on (address, shape, box) and is encoded once.
struct GenKey {
    const void* base; uint32_t rank; uint64_t dims[5]; uint64_t strides[4]; uint32_t box[5]; uint32_t swizzle;
    bool operator==(const GenKey& o) const {
        if (base != o.base || rank != o.rank || swizzle != o.swizzle) return false;
        for (int i = 0; i < 5; ++i) if (dims[i] != o.dims[i] || box[i] != o.box[i]) return false;
        for (int i = 0; i < 4; ++i) if (strides[i] != o.strides[i]) return false;
        return true;
    }
};
struct GenKeyHash {
    size_t operator()(const GenKey& k) const {
        size_t h = reinterpret_cast<size_t>(k.base) * 1000003u ^ k.rank ^ (k.swizzle << 8);
        for (int i = 0; i < 5; ++i) h = (h * 1000003u ^ k.dims[i]) * 31u ^ k.box[i];
        for (int i = 0; i < 4; ++i) h = h * 1000003u ^ k.strides[i];
        return h;
    }
};

// dims/box of dimension 0 in elements of `elem_bytes` (1, 2 or 4: a box may hold at most 256 elements per dimension, so wider
// elements allow wider boxes); strides are the byte strides of dimensions 1..rank-1.
int get_tensor_map_elems(const void* base, uint32_t elem_bytes, uint32_t rank, const uint64_t* dims, const uint64_t* strides, const uint32_t* box,
                         bool swizzle128, CUtensorMap* out) {
    static std::mutex mu;
    static std::unordered_map<GenKey, CUtensorMap, GenKeyHash> cache;
    GenKey k{};
    k.base = base; k.rank = rank; k.swizzle = (swizzle128 ? 1u : 0u) | (elem_bytes << 4);
    if (rank < 1 || rank > 5) return fail(TSP_E_ARG, "tensor map rank %u out of range", rank);
    if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4) return fail(TSP_E_ARG, "tensor map element size %u not supported", elem_bytes);
    for (uint32_t i = 0; i < 5; ++i) { k.dims[i] = i < rank ? dims[i] : 1; k.box[i] = i < rank ? box[i] : 1; }
    for (uint32_t i = 0; i < 4; ++i) k.strides[i] = i + 1 < rank ? strides[i] : 0;
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(k);
    if (it != cache.end()) { *out = it->second; return TSP_OK; }
    EncodeTiledFn enc = encode_fn();
    if (!enc) return fail(TSP_E_CUDA, "the CUDA driver does not export cuTensorMapEncodeTiled");
    cuuint64_t d[5], st[4];
    cuuint32_t b[5], es[5] = {1, 1, 1, 1, 1};
    for (uint32_t i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; }
    for (uint32_t i = 0; i + 1 < rank; ++i) st[i] = strides[i];
    const CUtensorMapDataType type = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32;
    CUtensorMap m;
    const CUresult r = enc(&m, type, rank, const_cast<void*>(base), d, st, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TSP_E_CUDA, "cuTensorMapEncodeTiled failed with %d", static_cast<int>(r));
    if (cache.size() > 4096) cache.clear();
    cache.emplace(k, m);
    *out = m;
    return TSP_OK;
}

// the same with byte elements
int get_tensor_map_bytes(const void* base, uint32_t rank, const uint64_t* dims, const uint64_t* strides, const uint32_t* box,
                         bool swizzle128, CUtensorMap* out) {
    return get_tensor_map_elems(base, 1, rank, dims, strides, box, swizzle128, out);
}

}  // namespace tsp
