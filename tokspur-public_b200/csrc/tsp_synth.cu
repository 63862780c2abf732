// Device-side data preparation: seeded synthetic weights quantised to GGUF Q4_K / Q8_0 blocks, and the
// GGUF -> Pack v3 planar repack (planar_pack_v3.cpp:676-716 restated per block, one thread per block).
// The generator stands in for a real model's weights at benchmark scale, where producing ~1 GB per
// layer on the host would dominate the run. Parity never depends on it: every check decodes the
// produced bytes with the oracle.
#include "tsp_common.cuh"

namespace tsp {

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    uint64_t z = x;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// element i of the N(0, sigma) stream `seed`: two counter-based uniforms, Box-Muller
__device__ __forceinline__ float normal_at(uint64_t key, uint64_t i, float sigma) {
    const uint64_t a = splitmix64((2 * i) * 0xD1342543DE82EF95ull + key);
    const uint64_t b = splitmix64((2 * i + 1) * 0xD1342543DE82EF95ull + key);
    const float u1 = (static_cast<float>(a >> 40) + 0.5f) * (1.0f / 16777216.0f);
    const float u2 = (static_cast<float>(b >> 40) + 0.5f) * (1.0f / 16777216.0f);
    return sigma * sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
}

// LEVELS 15: Q4_K (144-byte blocks, nibbles at byte 16); 31: Q5_K (176-byte blocks: the same header, 32 bytes of fifth bits, nibbles
// at byte 48; numeric.cpp:44-50)
template <int LEVELS>
__global__ void synth_q4k_kernel(uint64_t key, uint64_t first_block, uint64_t blocks, float sigma, uint8_t* __restrict__ out) {
    const uint64_t blk = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (blk >= blocks) return;
    const uint64_t e0 = (first_block + blk) * 256;
    float scale[8], minv[8];
    float max_scale = 0.f, max_min = 0.f;
    for (int g = 0; g < 8; ++g) {
        float lo = 0.f, hi = -INFINITY;
        for (int l = 0; l < 32; ++l) {
            const float v = normal_at(key, e0 + g * 32 + l, sigma);
            lo = fminf(lo, v);
            hi = fmaxf(hi, v);
        }
        minv[g] = -lo;
        scale[g] = (hi + minv[g]) / static_cast<float>(LEVELS);
        max_scale = fmaxf(max_scale, scale[g]);
        max_min = fmaxf(max_min, minv[g]);
    }
    const __half dh = __float2half_rn(max_scale / 63.0f), mh = __float2half_rn(max_min / 63.0f);
    const float d = __half2float(dh), dmin = __half2float(mh);
    uint8_t sc[8], mn[8];
    for (int g = 0; g < 8; ++g) {
        sc[g] = d > 0.f ? static_cast<uint8_t>(fminf(fmaxf(rintf(scale[g] / d), 0.f), 63.f)) : 0;
        mn[g] = dmin > 0.f ? static_cast<uint8_t>(fminf(fmaxf(rintf(minv[g] / dmin), 0.f), 63.f)) : 0;
    }
    constexpr bool Q5 = LEVELS == 31;
    uint8_t* b = out + blk * (Q5 ? 176 : 144);
    uint8_t* qs = b + (Q5 ? 48 : 16);
    if (Q5) for (int l = 0; l < 32; ++l) b[16 + l] = 0;
    const uint16_t db = __half_as_ushort(dh), mb = __half_as_ushort(mh);
    b[0] = db & 255; b[1] = db >> 8; b[2] = mb & 255; b[3] = mb >> 8;
    for (int g = 0; g < 4; ++g) {
        b[4 + g] = sc[g] | ((sc[g + 4] >> 4) << 6);
        b[8 + g] = mn[g] | ((mn[g + 4] >> 4) << 6);
        b[12 + g] = (sc[g + 4] & 15) | ((mn[g + 4] & 15) << 4);
    }
    for (int j = 0; j < 4; ++j) {
        const float dl0 = d * sc[2 * j], ml0 = dmin * mn[2 * j], dl1 = d * sc[2 * j + 1], ml1 = dmin * mn[2 * j + 1];
        for (int l = 0; l < 32; ++l) {
            const float v0 = normal_at(key, e0 + (2 * j) * 32 + l, sigma), v1 = normal_at(key, e0 + (2 * j + 1) * 32 + l, sigma);
            const uint32_t q0 = dl0 > 0.f ? static_cast<uint32_t>(fminf(fmaxf(rintf((v0 + ml0) / dl0), 0.f), static_cast<float>(LEVELS))) : 0u;
            const uint32_t q1 = dl1 > 0.f ? static_cast<uint32_t>(fminf(fmaxf(rintf((v1 + ml1) / dl1), 0.f), static_cast<float>(LEVELS))) : 0u;
            qs[j * 32 + l] = static_cast<uint8_t>((q0 & 15u) | ((q1 & 15u) << 4));
            if (Q5) b[16 + l] |= static_cast<uint8_t>(((q0 >> 4) << (2 * j)) | ((q1 >> 4) << (2 * j + 1)));
        }
    }
}

__global__ void synth_q8_kernel(uint64_t key, uint64_t first_block, uint64_t blocks, float sigma, uint8_t* __restrict__ out) {
    const uint64_t blk = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (blk >= blocks) return;
    const uint64_t e0 = (first_block + blk) * 32;
    float amax = 0.f;
    for (int l = 0; l < 32; ++l) amax = fmaxf(amax, fabsf(normal_at(key, e0 + l, sigma)));
    const __half dh = __float2half_rn(amax / 127.0f);
    const float d = __half2float(dh);
    uint8_t* b = out + blk * 34;
    const uint16_t db = __half_as_ushort(dh);
    b[0] = db & 255; b[1] = db >> 8;
    for (int l = 0; l < 32; ++l) {
        const float v = normal_at(key, e0 + l, sigma);
        const int q = d > 0.f ? static_cast<int>(fminf(fmaxf(rintf(v / d), -127.f), 127.f)) : 0;
        b[2 + l] = static_cast<uint8_t>(q & 255);
    }
}

// Q5_1: d = (max - min) / 31 and m = min as binary16, 32 fifth bits, 16 bytes of nibbles (numeric.cpp:38-42)
__global__ void synth_q51_kernel(uint64_t key, uint64_t first_block, uint64_t blocks, float sigma, uint8_t* __restrict__ out) {
    const uint64_t blk = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (blk >= blocks) return;
    const uint64_t e0 = (first_block + blk) * 32;
    float lo = INFINITY, hi = -INFINITY;
    for (int l = 0; l < 32; ++l) { const float v = normal_at(key, e0 + l, sigma); lo = fminf(lo, v); hi = fmaxf(hi, v); }
    const __half dh = __float2half_rn((hi - lo) / 31.0f), mh = __float2half_rn(lo);
    const float d = __half2float(dh), m = __half2float(mh);
    uint8_t* b = out + blk * 24;
    const uint16_t db = __half_as_ushort(dh), mb = __half_as_ushort(mh);
    b[0] = db & 255; b[1] = db >> 8; b[2] = mb & 255; b[3] = mb >> 8;
    uint32_t high = 0;
    uint8_t nib[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
    for (int l = 0; l < 32; ++l) {
        const float v = normal_at(key, e0 + l, sigma);
        const uint32_t q = d > 0.f ? static_cast<uint32_t>(fminf(fmaxf(rintf((v - m) / d), 0.f), 31.f)) : 0u;
        high |= (q >> 4) << l;
        nib[l & 15] |= static_cast<uint8_t>((q & 15u) << (4 * (l >> 4)));
    }
    b[4] = high & 255; b[5] = (high >> 8) & 255; b[6] = (high >> 16) & 255; b[7] = high >> 24;
    for (int i = 0; i < 16; ++i) b[8 + i] = nib[i];
}

__global__ void synth_f32_kernel(uint64_t key, uint64_t n, float sigma, float* __restrict__ out) {
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = normal_at(key, i, sigma);
}

// one thread per block of one expert; blocks_per_expert = rows * blocks_per_row
__global__ void pack_planar_kernel(uint32_t type, const uint8_t* __restrict__ gguf, uint64_t gguf_expert_stride,
                                   uint8_t* __restrict__ planar, uint64_t planar_expert_stride, uint64_t blocks_per_expert,
                                   uint32_t experts) {
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= blocks_per_expert * experts) return;
    const uint64_t e = i / blocks_per_expert, blk = i % blocks_per_expert;
    uint8_t* dst = planar + e * planar_expert_stride;
    if (type == TSP_TYPE_Q4_K) {
        const uint8_t* sb = gguf + e * gguf_expert_stride + blk * 144;
        const uint4* src = reinterpret_cast<const uint4*>(sb);
        uint4* q = reinterpret_cast<uint4*>(dst + blk * 128);
        for (int k = 0; k < 8; ++k) q[k] = src[1 + k];
        const uint8_t* s12 = sb + 4;
        uint8_t* sm = dst + blocks_per_expert * 128 + blk * 16;
        for (int s = 0; s < 4; ++s) {
            sm[s] = s12[s] & 0x3f;
            sm[4 + s] = (s12[8 + s] & 0x0f) | ((s12[s] >> 6) << 4);
            sm[8 + s] = s12[4 + s] & 0x3f;
            sm[12 + s] = (s12[8 + s] >> 4) | ((s12[4 + s] >> 6) << 4);
        }
        *reinterpret_cast<uint32_t*>(dst + blocks_per_expert * 144 + blk * 4) = *reinterpret_cast<const uint32_t*>(sb);
    } else {
        const uint8_t* sb = gguf + e * gguf_expert_stride + blk * 34;
        uint8_t* q = dst + blk * 32;
        for (int k = 0; k < 32; ++k) q[k] = sb[2 + k];
        uint8_t* dm = dst + blocks_per_expert * 32 + blk * 2;
        dm[0] = sb[0]; dm[1] = sb[1];
    }
}

int launch_synth(uint32_t type, uint64_t seed, uint64_t first_block, uint64_t blocks, float sigma, void* out, cudaStream_t st) {
    const uint64_t key = seed * 0x9E3779B97F4A7C15ull + 0x632BE59BD9B4E019ull;
    const unsigned grid = static_cast<unsigned>((blocks + 127) / 128);
    if (type == TSP_TYPE_Q4_K) synth_q4k_kernel<15><<<grid, 128, 0, st>>>(key, first_block, blocks, sigma, static_cast<uint8_t*>(out));
    else if (type == TSP_TYPE_Q5_K) synth_q4k_kernel<31><<<grid, 128, 0, st>>>(key, first_block, blocks, sigma, static_cast<uint8_t*>(out));
    else if (type == TSP_TYPE_Q5_1) synth_q51_kernel<<<grid, 128, 0, st>>>(key, first_block, blocks, sigma, static_cast<uint8_t*>(out));
    else if (type == TSP_TYPE_Q8_0) synth_q8_kernel<<<grid, 128, 0, st>>>(key, first_block, blocks, sigma, static_cast<uint8_t*>(out));
    else synth_f32_kernel<<<grid, 128, 0, st>>>(key, blocks, sigma, static_cast<float*>(out));
    TSP_CUDA(cudaGetLastError());
    return TSP_OK;
}

int launch_pack_planar(uint32_t type, const void* gguf, uint64_t gguf_stride, void* planar, uint64_t planar_stride,
                       uint64_t blocks_per_expert, uint32_t experts, cudaStream_t st) {
    const uint64_t total = blocks_per_expert * experts;
    pack_planar_kernel<<<static_cast<unsigned>((total + 127) / 128), 128, 0, st>>>(
        type, static_cast<const uint8_t*>(gguf), gguf_stride, static_cast<uint8_t*>(planar), planar_stride, blocks_per_expert, experts);
    TSP_CUDA(cudaGetLastError());
    return TSP_OK;
}

// ---------------------------------------------------------------------------------------------
// `q8_lanes_v1` rows <-> GGUF Q8_0 rows (expert_lanes.cpp:75-130), a lossless re-layout done once when a tensor is loaded: the
// Pack v3 container stores dense Q8_0 matrices (the vocabulary head among them) in the lane layout, the kernels here read
// GGUF rows. One block of threads per (row, run of up to 16 quant blocks): the run's 512 code bytes pass through shared memory.
// ---------------------------------------------------------------------------------------------
template <bool UNPACK>
__global__ void __launch_bounds__(128) q8_lanes_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, uint32_t blocks) {
    __shared__ uint8_t codes[512];
    const uint64_t row = blockIdx.y;
    const uint32_t run = blockIdx.x, tid = threadIdx.x;
    const uint32_t width = min(16u, blocks - run * 16u);           // blocks in this run
    const uint64_t row_bytes = static_cast<uint64_t>(blocks) * 34u;
    const uint8_t* src = in + row * row_bytes;
    uint8_t* dst = out + row * row_bytes;
    const uint32_t meta = blocks * 2u;
    if (UNPACK) {
        // lanes: scales at 2 b, code i of block b at meta + run*512 + i*width + b%16
        for (uint32_t k = tid; k < width * 32u; k += 128) codes[k] = src[meta + run * 512u + k];
        __syncthreads();
        for (uint32_t k = tid; k < width * 17u; k += 128) {        // 17 half-words per GGUF block
            const uint32_t b = k / 17u, h = k % 17u, blk = run * 16u + b;
            uint16_t v;
            if (h == 0) v = *reinterpret_cast<const uint16_t*>(src + blk * 2u);
            else v = static_cast<uint16_t>(codes[(2 * h - 2) * width + b]) | (static_cast<uint16_t>(codes[(2 * h - 1) * width + b]) << 8);
            *reinterpret_cast<uint16_t*>(dst + blk * 34u + h * 2u) = v;
        }
    } else {
        for (uint32_t k = tid; k < width * 17u; k += 128) {
            const uint32_t b = k / 17u, h = k % 17u, blk = run * 16u + b;
            const uint16_t v = *reinterpret_cast<const uint16_t*>(src + blk * 34u + h * 2u);
            if (h == 0) *reinterpret_cast<uint16_t*>(dst + blk * 2u) = v;
            else { codes[(2 * h - 2) * width + b] = static_cast<uint8_t>(v); codes[(2 * h - 1) * width + b] = static_cast<uint8_t>(v >> 8); }
        }
        __syncthreads();
        for (uint32_t k = tid; k < width * 32u; k += 128) dst[meta + run * 512u + k] = codes[k];
    }
}

int launch_q8_lanes(const void* in, void* out, uint64_t rows, uint32_t cols, bool unpack, cudaStream_t st) {
    const uint32_t blocks = cols / 32u;
    for (uint64_t r0 = 0; r0 < rows; r0 += 65535) {   // grid.y limit
        const uint32_t n = static_cast<uint32_t>(rows - r0 < 65535 ? rows - r0 : 65535);
        const dim3 grid((blocks + 15u) / 16u, n);
        const uint8_t* src = static_cast<const uint8_t*>(in) + r0 * blocks * 34ull;
        uint8_t* dst = static_cast<uint8_t*>(out) + r0 * blocks * 34ull;
        if (unpack) q8_lanes_kernel<true><<<grid, 128, 0, st>>>(src, dst, blocks);
        else q8_lanes_kernel<false><<<grid, 128, 0, st>>>(src, dst, blocks);
    }
    TSP_CUDA(cudaGetLastError());
    return TSP_OK;
}

}  // namespace tsp
