// Top-64 rows of the sampler behind the vocabulary head: replaces the reference's `MetalGraph::logit_topk` (graph.mm:9443-9478,
// two dispatches `logit_topk_stage1` / `logit_topk_stage2`; row type `GpuLogitTopKRow`, sampling.hpp:21-29; CPU statement
// `cpu_logit_topk_row`, sampling.cpp:473-515).
//
// Order: value descending with -0 == +0, ties to the lower column; non-finite logits are left out (first such column recorded),
// the first subnormal column is recorded while the value still competes; the raw bits of the logits are returned.
//
// Both stages find their 64 winners with a radix select over keys that are unique by construction (value bits above, inverted
// column below), so the set is exact and no tie needs a second rule; the winners are then ranked by counting. Stage 1 works on
// tiles of 4096 columns (one block each), stage 2 merges the tiles' rows (one block per logits row).
#include "tsp_common.cuh"

namespace tsp {

constexpr int kTopkThreads = 256;
constexpr uint32_t kTopkCap = TSP_TOPK_CAPACITY, kTopkSpan = TSP_TOPK_TILE_SPAN;
constexpr uint32_t kTopkRowWords = 4 + 2 * kTopkCap;   // 528 bytes

// Order-preserving 32-bit image of a finite logit (-0 counted as +0): larger value -> larger image, never below 0x00800000.
__device__ __forceinline__ uint32_t topk_mono(float v) {
    uint32_t b = __float_as_uint(v);
    if ((b << 1) == 0) b = 0;
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct TopkShared {
    uint32_t hist[256];
    unsigned long long sel[kTopkCap];
    uint32_t digit, need, whole, taken, nonfinite, subnormal, valid;
};

// A lower bound T such that exactly `need` of the block's keys (all distinct, 0 = no key, `bits` wide) are >= T, found digit by
// digit (8 bits) from the top with a shared-memory histogram; the walk stops as soon as the digit's bucket is needed whole,
// which for spread-out values is after two or three digits. Measured alternatives on 4096-column tiles: one warp-aggregated
// atomic per distinct digit (`match.any`), a bit-by-bit walk without atomics and a start below the keys' common prefix (an extra
// max / min reduction) were all slower (40 / 39 / 32 us against 28 us for 16 rows of 151 936 logits). each(f) calls f(key) for every key of the calling thread. All threads return the same value.
// sh.hist must be zero on entry and is zero again on return.
template <class Each>
__device__ unsigned long long topk_select(TopkShared& sh, Each each, uint32_t need, int bits) {
    const uint32_t tid = threadIdx.x, lane = tid & 31;
    unsigned long long prefix = 0;
    int done = 0;   // bits already fixed
    while (done < bits) {
        const int width = bits - done >= 8 ? 8 : bits - done, shift = bits - done - width;
        each([&](unsigned long long key) {
            if (key != 0 && (key >> (shift + width)) == prefix) atomicAdd(&sh.hist[static_cast<uint32_t>(key >> shift) & ((1u << width) - 1u)], 1u);
        });
        __syncthreads();
        if (tid < 32) {
            // lane l holds digits 8l .. 8l+7; walk from the top digit down until `need` keys are covered
            uint32_t c[8], mine = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) { c[i] = sh.hist[lane * 8 + i]; sh.hist[lane * 8 + i] = 0; mine += c[i]; }
            uint32_t suffix = mine;   // keys in the lanes at and above this one
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t v = __shfl_down_sync(0xffffffffu, suffix, o);
                if (lane + o < 32) suffix += v;
            }
            uint32_t acc = suffix - mine;
            if (acc < need && suffix >= need) {
#pragma unroll
                for (int i = 7; i >= 0; --i) {
                    if (acc < need && acc + c[i] >= need) { sh.digit = lane * 8 + i; sh.need = need - acc; sh.whole = (need - acc == c[i]); }
                    acc += c[i];
                }
            }
        }
        __syncthreads();
        prefix = (prefix << width) | sh.digit;
        need = sh.need;
        done += width;
        if (sh.whole) break;   // every key of this bucket is wanted: the bucket's lowest possible key is the bound
    }
    return prefix << (bits - done);
}

// Appends the keys at or above the bound to sh.sel: one shared-memory atomic per warp and call instead of one per key (the
// per-key form serialised 64 atomics on one counter: 2.2 k cycles). Must be called by whole warps.
__device__ __forceinline__ void topk_take(TopkShared& sh, unsigned long long key, unsigned long long threshold) {
    const bool take = key >= threshold && key != 0;
    const uint32_t votes = __ballot_sync(0xffffffffu, take);
    if (!votes) return;
    const uint32_t lane = threadIdx.x & 31, leader = __ffs(votes) - 1;
    uint32_t at = 0;
    if (lane == leader) at = atomicAdd(&sh.taken, static_cast<uint32_t>(__popc(votes)));
    at = __shfl_sync(0xffffffffu, at, leader);
    if (take) sh.sel[at + __popc(votes & ((1u << lane) - 1u))] = key;
}

// Ranks the sh.taken (<= 64) selected keys by counting and returns this thread's key for output slot tid (0 if none).
__device__ unsigned long long topk_ranked(TopkShared& sh, unsigned long long* ranked) {
    const uint32_t tid = threadIdx.x;
    if (tid < kTopkCap) ranked[tid] = 0;
    __syncthreads();
    if (tid < sh.taken) {
        const unsigned long long mine = sh.sel[tid];
        uint32_t rank = 0;
        for (uint32_t i = 0; i < sh.taken; ++i) rank += sh.sel[i] > mine;
        ranked[rank] = mine;
    }
    __syncthreads();
    return tid < kTopkCap ? ranked[tid] : 0ull;
}

__global__ void __launch_bounds__(kTopkThreads)
logit_topk_tiles_kernel(const float* __restrict__ logits, uint64_t stride, uint32_t vocabulary, uint32_t tiles, uint32_t* __restrict__ partial) {
    pdl_launch_dependents();
    __shared__ TopkShared sh;
    __shared__ unsigned long long ranked[kTopkCap];
    const uint32_t tid = threadIdx.x, tile = blockIdx.x, row = blockIdx.y;
    const uint32_t base = tile * kTopkSpan;
    sh.hist[tid] = 0;
    if (tid == 0) { sh.nonfinite = sh.subnormal = 0xffffffffu; sh.valid = 0; sh.taken = 0; }
    __syncthreads();
    pdl_wait();
    const float* src = reinterpret_cast<const float*>(reinterpret_cast<const char*>(logits) + row * stride);
    // 16 columns per thread, key = value image above 12 bits of inverted position inside the tile (44 bits)
    unsigned long long k[16];
    uint32_t valid = 0, nonfinite = 0xffffffffu, subnormal = 0xffffffffu;
    float vals[16];
#pragma unroll
    for (uint32_t i = 0; i < 16; ++i) {   // all loads first: sixteen dependent round trips otherwise (measured 6.8 k cycles of a 19 k block)
        const uint32_t col = base + i * kTopkThreads + tid;
        vals[i] = src[min(col, vocabulary - 1)];
    }
#pragma unroll
    for (uint32_t i = 0; i < 16; ++i) {
        const uint32_t local = i * kTopkThreads + tid, col = base + local;
        k[i] = 0;
        if (col < vocabulary) {
            const float v = vals[i];
            const uint32_t b = __float_as_uint(v);
            if ((b & 0x7f800000u) == 0x7f800000u) { nonfinite = min(nonfinite, col); continue; }
            if ((b & 0x7f800000u) == 0 && (b & 0x007fffffu)) subnormal = min(subnormal, col);
            k[i] = (static_cast<unsigned long long>(topk_mono(v)) << 12) | (4095u - local);
            ++valid;
        }
    }
    if (nonfinite != 0xffffffffu) atomicMin(&sh.nonfinite, nonfinite);
    if (subnormal != 0xffffffffu) atomicMin(&sh.subnormal, subnormal);
    if (valid) atomicAdd(&sh.valid, valid);
    __syncthreads();
    const uint32_t count = min(sh.valid, kTopkCap);
    auto each = [&](auto f) {
#pragma unroll
        for (uint32_t i = 0; i < 16; ++i) f(k[i]);
    };
    if (count) {
        const unsigned long long threshold = topk_select(sh, each, count, 44);
        each([&](unsigned long long key) { topk_take(sh, key, threshold); });
        __syncthreads();
    }
    const unsigned long long mine = topk_ranked(sh, ranked);
    uint32_t* out = partial + (static_cast<uint64_t>(row) * tiles + tile) * kTopkRowWords;
    if (tid == 0) { out[0] = vocabulary; out[1] = count; out[2] = sh.nonfinite; out[3] = sh.subnormal; }
    if (tid < kTopkCap) {
        uint32_t id = 0;
        float v = -INFINITY;
        if (mine) { id = base + 4095u - static_cast<uint32_t>(mine & 4095u); v = src[id]; }
        out[4 + tid] = id;
        out[4 + kTopkCap + tid] = __float_as_uint(v);
    }
}

template <bool REGS>
__global__ void __launch_bounds__(kTopkThreads)
logit_topk_merge_kernel(const uint32_t* __restrict__ partial, uint32_t vocabulary, uint32_t tiles, uint32_t* __restrict__ rows_out) {
    pdl_launch_dependents();
    __shared__ TopkShared sh;
    __shared__ unsigned long long ranked[kTopkCap];
    const uint32_t tid = threadIdx.x, row = blockIdx.x;
    sh.hist[tid] = 0;
    if (tid == 0) { sh.nonfinite = sh.subnormal = 0xffffffffu; sh.valid = 0; sh.taken = 0; }
    __syncthreads();
    pdl_wait();
    const uint32_t* src = partial + static_cast<uint64_t>(row) * tiles * kTopkRowWords;
    uint32_t valid = 0, nonfinite = 0xffffffffu, subnormal = 0xffffffffu;
    for (uint32_t t = tid; t < tiles; t += kTopkThreads) {
        const uint32_t* h = src + static_cast<uint64_t>(t) * kTopkRowWords;
        valid += min(h[1], kTopkCap); nonfinite = min(nonfinite, h[2]); subnormal = min(subnormal, h[3]);
    }
    if (nonfinite != 0xffffffffu) atomicMin(&sh.nonfinite, nonfinite);
    if (subnormal != 0xffffffffu) atomicMin(&sh.subnormal, subnormal);
    if (valid) atomicAdd(&sh.valid, valid);
    __syncthreads();
    const uint32_t count = min(sh.valid, kTopkCap);
    // candidates: slot s of tile t is live when s < that tile's count; key = value image above the inverted column (64 bits)
    const uint32_t cands = tiles * kTopkCap;
    auto key_at = [&](uint32_t i) -> unsigned long long {
        const uint32_t t = i / kTopkCap, s = i % kTopkCap;
        const uint32_t* h = src + static_cast<uint64_t>(t) * kTopkRowWords;
        const uint32_t live = h[1], id = h[4 + s], bits = h[4 + kTopkCap + s];   // three independent loads (every slot of a row exists)
        if (s >= min(live, kTopkCap)) return 0ull;
        return (static_cast<unsigned long long>(topk_mono(__uint_as_float(bits))) << 32) | (0xffffffffu - id);
    };
    if (REGS) {   // up to 64 tiles: the candidates are read once, 16 per thread, and the digit walk runs out of registers
        unsigned long long k[16];
#pragma unroll
        for (uint32_t i = 0; i < 16; ++i) { const uint32_t c = i * kTopkThreads + tid; k[i] = c < cands ? key_at(c) : 0ull; }
        auto each = [&](auto f) {
#pragma unroll
            for (uint32_t i = 0; i < 16; ++i) f(k[i]);
        };
        if (count) {
            const unsigned long long threshold = topk_select(sh, each, count, 64);
            each([&](unsigned long long key) { topk_take(sh, key, threshold); });
            __syncthreads();
        }
    } else {
        auto each = [&](auto f) { for (uint32_t i = tid; i < cands; i += kTopkThreads) f(key_at(i)); };
        if (count) {
            const unsigned long long threshold = topk_select(sh, each, count, 64);
            each([&](unsigned long long key) { topk_take(sh, key, threshold); });
            __syncthreads();
        }
    }
    const unsigned long long mine = topk_ranked(sh, ranked);
    uint32_t* out = rows_out + static_cast<uint64_t>(row) * kTopkRowWords;
    if (tid == 0) { out[0] = vocabulary; out[1] = count; out[2] = sh.nonfinite; out[3] = sh.subnormal; }
    if (tid < kTopkCap) {
        uint32_t id = 0, bits = 0xff800000u;   // -infinity
        if (mine) {
            id = 0xffffffffu - static_cast<uint32_t>(mine & 0xffffffffu);
            // the raw bits (a -0 keeps its sign) sit in the tile's row next to the id
            const uint32_t* h = src + static_cast<uint64_t>(id / kTopkSpan) * kTopkRowWords;
            for (uint32_t s = 0; s < kTopkCap; ++s) if (h[4 + s] == id && s < h[1]) { bits = h[4 + kTopkCap + s]; break; }
        }
        out[4 + tid] = id;
        out[4 + kTopkCap + tid] = bits;
    }
}

int launch_logit_topk(const float* logits, uint64_t stride, uint32_t rows, uint32_t vocabulary, uint32_t* partial, uint32_t* out, cudaStream_t st) {
    const uint32_t tiles = (vocabulary + kTopkSpan - 1) / kTopkSpan;
    TSP_CUDA(launch_pdl(logit_topk_tiles_kernel, dim3(tiles, rows), dim3(kTopkThreads), 0, st, logits, stride, vocabulary, tiles, partial));
    if (tiles <= 64) TSP_CUDA(launch_pdl(logit_topk_merge_kernel<true>, dim3(rows), dim3(kTopkThreads), 0, st, static_cast<const uint32_t*>(partial), vocabulary, tiles, out));
    else TSP_CUDA(launch_pdl(logit_topk_merge_kernel<false>, dim3(rows), dim3(kTopkThreads), 0, st, static_cast<const uint32_t*>(partial), vocabulary, tiles, out));
    TSP_CUDA(cudaGetLastError());
    return TSP_OK;
}

}  // namespace tsp
