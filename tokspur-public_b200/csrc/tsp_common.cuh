// Shared device helpers for the sm_100a MoE kernels: binary16 decode, error word, mbarrier and
// bulk-copy (TMA) PTX wrappers with bounded waits.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tsp_moe.h"

namespace tsp {

// ---------------------------------------------------------------------------------------------
// host-side error reporting (thread-local message behind tsp_last_error)
// ---------------------------------------------------------------------------------------------
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
#define TSP_REQUIRE(cond, ...) do { if (!(cond)) return ::tsp::fail(TSP_E_ARG, __VA_ARGS__); } while (0)
#define TSP_CUDA(expr) do { cudaError_t e_ = (expr); if (e_ != cudaSuccess) return ::tsp::cuda_fail(e_, #expr); } while (0)
int sm_count();  // SM count of the current device (cached), 0 when no device is usable

// kernel<<<grid, block, smem, stream>>>(args...) with programmatic stream serialisation allowed (see pdl_wait below)
template <typename... Params, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

// A dense expert (experts == 1 sets with the routed experts' shape, encoding and layout) that a routed projection launch
// also processes, for every token row: input rows `x`, output rows `out`. b is used by gate-up launches only.
struct GemvShared {
    const tsp_matrix_set* a; const tsp_matrix_set* b;
    const float* x; uint64_t x_stride_bytes;
    float* out; uint64_t out_stride_bytes;
    // optional: the token rows as binary16 (exactly the values of `x`); both the routed and the dense tiles then read these
    const void* x16 = nullptr; uint64_t x16_stride_bytes = 0;
    uint32_t tokens = 0;   // rows of the dense expert (0: as many as the routed launch has token rows)
};

// the layer's dense shared expert riding in a routed launch: one-expert matrix sets of the routed experts' shape, binary16
// activation rows of all `tokens` rows in row order, output rows in row order
struct GroupedShared {
    const tsp_matrix_set* a; const tsp_matrix_set* b;
    const void* act; uint64_t act_stride; uint32_t tokens;
    void* out; uint64_t out_stride;
};

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-DEVICE property of a kernel: what has been set on one device says
// nothing about the next one. Every launcher keeps one of these per kernel instantiation and asks it before a launch.
struct SmemAttrCache {
    static constexpr int kDevices = 64;
    size_t bytes[kDevices] = {};
    // true when `smem` exceeds what is known to be configured for `device` (the caller then sets the attribute and calls note())
    bool needs(int device, size_t smem) const { return device < 0 || device >= kDevices || smem > bytes[device]; }
    void note(int device, size_t smem) { if (device >= 0 && device < kDevices && smem > bytes[device]) bytes[device] = smem; }
};
template <typename Kernel>
static inline cudaError_t ensure_dynamic_smem(Kernel kernel, SmemAttrCache& cache, size_t smem) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (!cache.needs(dev, smem)) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e == cudaSuccess) cache.note(dev, smem);
    return e;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---------------------------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void raise_error(uint32_t* error, uint32_t bits) {
    if (error) atomicOr(error, bits);
}

__device__ __forceinline__ float half_bits_to_float(uint32_t bits16) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(bits16)));
}

__device__ __forceinline__ bool finite_f32(float v) { return (__float_as_uint(v) & 0x7f800000u) != 0x7f800000u; }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// ---- mbarrier -------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls and returns false; the caller raises TSP_ERR_TIMEOUT and
// leaves its loop, so a lost arrival can never hang the device.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 24)) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(32);
    }
    return false;
}

// ---- bulk asynchronous copy global -> shared (TMA, untiled form) -------------------------------
// Both addresses 16-byte aligned, size a multiple of 16 bytes. Completion is signalled on `bar`
// as transaction bytes.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// ---- programmatic dependent launch -------------------------------------------------------------
// Every kernel of the layer is launched with programmatic stream serialisation allowed: its launch is processed while the
// previous kernel of the stream still runs, which hides the launch latency between the layer's short kernels. The
// contract kept by every kernel here: `pdl_launch_dependents()` first (the next kernel may then be scheduled once all CTAs
// of this one have started), set-up that touches no global memory, then `pdl_wait()` on every path before the first
// global access; the wait returns when the previous kernel has completed and its writes are visible, so the chain of
// kernels stays transitively ordered.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- named barrier among a subset of warps ---------------------------------------------------
__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---- legacy warp MMA used by the decode-size kernels: D(16x8,f32) += A(16x16,f16) * B(16x8,f16) ----
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// same with a zero accumulator input (no register initialisation needed)
__device__ __forceinline__ void mma_f16_16816_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                   uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// Branch-stable sigmoid / SiLU in FP32 (operators.cpp:28-36 restated for float).
__device__ __forceinline__ float stable_sigmoid(float v) {
    if (v >= 0.f) return 1.f / (1.f + expf(-v));
    const float p = expf(v);
    return p / (1.f + p);
}
__device__ __forceinline__ float stable_silu(float v) { return v * stable_sigmoid(v); }

}  // namespace tsp
