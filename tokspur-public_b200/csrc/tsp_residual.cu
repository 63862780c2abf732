// Hyper-connection residual read / write: the step either side of the MoE FFN sub-layer in every layer
// (MetalGraph::residual_read / residual_write, native/include/tokspur/graph.hpp:1056-1058; CPU forms operators.cpp:60-96).
// Element-wise FP32 work over [tokens][branches][channels] rows: bound by HBM bandwidth, one pass each.
#include "tsp_common.cuh"

namespace tsp {

// out[t][c] = sum_b normalized[t][b][c] * sigmoid(scores[t][b][c]) / branches      (branch order ascending, as the reference adds them)
// scales[t][b] = 2 * sigmoid(inject_logits[t][b] / branches)
__global__ void __launch_bounds__(256)
residual_read_kernel(const float* __restrict__ normalized, const float* __restrict__ scores, const float* __restrict__ inject_logits,
                     uint32_t branches, uint32_t channels, float* __restrict__ output, float* __restrict__ scales, uint32_t* error) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t t = blockIdx.y;
    const uint64_t row = static_cast<uint64_t>(t) * branches * channels;
    const float inv = 1.f / static_cast<float>(branches);
    bool bad = false;
    for (uint32_t c = blockIdx.x * blockDim.x + threadIdx.x; c < channels; c += gridDim.x * blockDim.x) {
        float acc = 0.f;
        for (uint32_t b = 0; b < branches; ++b) {
            const uint64_t at = row + static_cast<uint64_t>(b) * channels + c;
            acc += normalized[at] * stable_sigmoid(scores[at]) * inv;
        }
        bad |= !finite_f32(acc);
        output[static_cast<uint64_t>(t) * channels + c] = acc;
    }
    if (blockIdx.x == 0 && threadIdx.x < branches) {
        const float s = 2.f * stable_sigmoid(inject_logits[static_cast<uint64_t>(t) * branches + threadIdx.x] * inv);
        bad |= !finite_f32(s);
        scales[static_cast<uint64_t>(t) * branches + threadIdx.x] = s;
    }
    if (bad) raise_error(error, TSP_ERR_NONFINITE);
}

// destination[t][b][c] = streams[t][b][c] + scales[t][b] * output[t][c]
__global__ void __launch_bounds__(256)
residual_write_kernel(const float* __restrict__ streams, const float* __restrict__ output, const float* __restrict__ scales, uint32_t branches,
                      uint32_t channels, float* __restrict__ destination, uint32_t* error) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t t = blockIdx.y;
    const uint64_t row = static_cast<uint64_t>(t) * branches * channels;
    bool bad = false;
    for (uint32_t c = blockIdx.x * blockDim.x + threadIdx.x; c < channels; c += gridDim.x * blockDim.x) {
        const float o = output[static_cast<uint64_t>(t) * channels + c];
        for (uint32_t b = 0; b < branches; ++b) {
            const uint64_t at = row + static_cast<uint64_t>(b) * channels + c;
            const float v = fmaf(scales[static_cast<uint64_t>(t) * branches + b], o, streams[at]);
            bad |= !finite_f32(v);
            destination[at] = v;
        }
    }
    if (bad) raise_error(error, TSP_ERR_NONFINITE);
}

int launch_residual_read(const float* normalized, const float* scores, const float* inject_logits, uint32_t branches, uint32_t channels,
                         uint32_t tokens, float* output, float* scales, uint32_t* error, cudaStream_t st) {
    const dim3 grid((channels + 255) / 256, tokens);
    TSP_CUDA(launch_pdl(residual_read_kernel, grid, dim3(256), 0, st, normalized, scores, inject_logits, branches, channels, output, scales, error));
    return TSP_OK;
}

int launch_residual_write(const float* streams, const float* output, const float* scales, uint32_t branches, uint32_t channels, uint32_t tokens,
                          float* destination, uint32_t* error, cudaStream_t st) {
    const dim3 grid((channels + 255) / 256, tokens);
    TSP_CUDA(launch_pdl(residual_write_kernel, grid, dim3(256), 0, st, streams, output, scales, branches, channels, destination, error));
    return TSP_OK;
}

}  // namespace tsp
