// Router top-k, stable token permutation, gated combine and the activation edge conversions.
// All integer results (ids, token_map, counts, tasks) are deterministic and independent of
// scheduling: no atomics decide an order anywhere.
#include "tsp_common.cuh"

namespace tsp {

// ---------------------------------------------------------------------------------------------
// route: one warp per token row. Selection order is (logit descending, id ascending), i.e. the
// total order of route_reference (routing.cpp:15-18). Logits are compared as FP32, which orders
// exactly as the reference's doubles do because the conversion is exact.
// Weights are evaluated in double so that they round to the same FP32 as the reference's.
// ---------------------------------------------------------------------------------------------
constexpr int kRouteWarps = 4;  // at most; fewer when a row of logits is long, to stay inside 48 KB of shared memory

__device__ __forceinline__ double softplus_f64(double v) { return fmax(v, 0.0) + log1p(exp(-fabs(v))); }
__device__ __forceinline__ double sigmoid_f64(double v) {
    if (v >= 0) return 1.0 / (1.0 + exp(-v));
    const double p = exp(v);
    return p / (1.0 + p);
}

// One warp routes one token row; `row` is the warp's scratch of `experts` floats in shared memory.
// `margins` (optional): margins[token] = logit of the last selected expert - logit of the best expert left out (+inf when every
// expert is selected): how far the selection is from changing under a perturbation of the logits.
__device__ __forceinline__ void route_row(float* row, const float* __restrict__ src, uint32_t token, uint32_t experts, uint32_t selected,
                                          uint32_t mode, int normalize, uint32_t* __restrict__ ids, float* __restrict__ weights,
                                          uint32_t* error, uint32_t lane, float* __restrict__ margins = nullptr) {
    bool bad = false;
    for (uint32_t e = lane; e < experts; e += 32) {
        const float v = src[e];
        bad |= !finite_f32(v);
        row[e] = v;
    }
    bad = __any_sync(0xffffffffu, bad);
    __syncwarp();
    uint32_t* out_ids = ids + static_cast<uint64_t>(token) * selected;
    float* out_w = weights + static_cast<uint64_t>(token) * selected;
    if (bad) {  // reference: FormatError("nonfinite router logit"); here: flag and publish a harmless row
        if (lane == 0) raise_error(error, TSP_ERR_NONFINITE);
        for (uint32_t r = lane; r < selected; r += 32) { out_ids[r] = r; out_w[r] = 0.f; }
        if (margins && lane == 0) margins[token] = 0.f;
        return;
    }
    // full-softmax denominator (only when not renormalising over the selection)
    double all_sum = 0;
    float row_max = -INFINITY;
    for (uint32_t e = lane; e < experts; e += 32) row_max = fmaxf(row_max, row[e]);
    for (int o = 16; o; o >>= 1) row_max = fmaxf(row_max, __shfl_xor_sync(0xffffffffu, row_max, o));
    if (mode == TSP_ROUTER_SOFTMAX && !normalize) {
        // ascending-id order of additions as in the reference loop, made deterministic by a serial lane-0 pass
        if (lane == 0) for (uint32_t e = 0; e < experts; ++e) all_sum += exp(static_cast<double>(row[e]) - static_cast<double>(row_max));
        all_sum = __shfl_sync(0xffffffffu, all_sum, 0);
    }
    // lane r keeps the logit of rank r (ranks >= 32 in a second slot); the double-precision activations are then
    // evaluated once per rank, in parallel across lanes, instead of once per rank by every lane
    float my_logit = 0.f, my_logit_hi = 0.f;
    for (uint32_t r = 0; r < selected; ++r) {
        float best = -INFINITY;
        uint32_t best_id = 0xffffffffu;
        for (uint32_t e = lane; e < experts; e += 32) {
            const float v = row[e];
            if (v > best) { best = v; best_id = e; }  // ascending scan keeps the lowest id on ties
        }
        for (int o = 16; o; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, best_id, o);
            if (ov > best || (ov == best && oi < best_id)) { best = ov; best_id = oi; }
        }
        if ((r & 31u) == lane) { if (r < 32) my_logit = best; else my_logit_hi = best; }
        if (lane == 0) { out_ids[r] = best_id; row[best_id] = -INFINITY; }
        __syncwarp();
    }
    if (margins) {   // one more round: the best logit among the experts left out
        float next = -INFINITY;
        for (uint32_t e = lane; e < experts; e += 32) next = fmaxf(next, row[e]);
        for (int o = 16; o; o >>= 1) next = fmaxf(next, __shfl_xor_sync(0xffffffffu, next, o));
        const uint32_t last = selected - 1;
        const float last_logit = __shfl_sync(0xffffffffu, last < 32 ? my_logit : my_logit_hi, last & 31u);
        if (lane == 0) margins[token] = selected < experts ? last_logit - next : INFINITY;
    }
    const double mx = row_max;
    auto activate = [&](float logit) -> double {
        const double l = logit;
        if (mode == TSP_ROUTER_SOFTMAX) return exp(l - mx);
        if (normalize) return exp(-softplus_f64(-l) + softplus_f64(-mx));
        return sigmoid_f64(l);
    };
    const double my_act = lane < selected ? activate(my_logit) : 0.0;
    const double my_act_hi = lane + 32 < selected ? activate(my_logit_hi) : 0.0;
    double sel_sum = my_act + my_act_hi;   // fixed butterfly order: deterministic, within an ulp of the rank-order sum
    for (int o = 16; o; o >>= 1) sel_sum += __shfl_xor_sync(0xffffffffu, sel_sum, o);
    double denominator = mode == TSP_ROUTER_SIGMOID ? 1.0 : all_sum;
    if (normalize) denominator = sel_sum;
    if (!(denominator > 0) || isinf(denominator)) {
        if (lane == 0) raise_error(error, TSP_ERR_NONFINITE);
        denominator = 1.0;
    }
    if (lane < selected) out_w[lane] = static_cast<float>(my_act / denominator);
    if (lane + 32 < selected) out_w[lane + 32] = static_cast<float>(my_act_hi / denominator);
}

// The same selection for rows of at most 512 logits kept in registers (expert e = lane + 32 i in slot i), used where one block
// routes a whole decode batch: about a fifth of the instructions of the shared-memory form. Same total order (value descending,
// id ascending), same double-precision weights. Full-softmax weights without renormalisation need the serial ascending-id sum
// and stay with route_row.
__device__ __forceinline__ void route_row_regs(const float* __restrict__ src, uint32_t token, uint32_t experts, uint32_t selected,
                                               uint32_t mode, uint32_t* __restrict__ ids, float* __restrict__ weights, uint32_t* error,
                                               uint32_t lane) {
    float v[16];
    bool bad = false;
#pragma unroll
    for (uint32_t i = 0; i < 16; ++i) {
        const uint32_t e = lane + 32 * i;
        v[i] = e < experts ? src[e] : -INFINITY;
        bad |= e < experts && !finite_f32(v[i]);
    }
    bad = __any_sync(0xffffffffu, bad);
    uint32_t* out_ids = ids + static_cast<uint64_t>(token) * selected;
    float* out_w = weights + static_cast<uint64_t>(token) * selected;
    if (bad) {
        if (lane == 0) raise_error(error, TSP_ERR_NONFINITE);
        for (uint32_t r = lane; r < selected; r += 32) { out_ids[r] = r; out_w[r] = 0.f; }
        return;
    }
    float row_max = -INFINITY;
#pragma unroll
    for (uint32_t i = 0; i < 16; ++i) row_max = fmaxf(row_max, v[i]);
    for (int o = 16; o; o >>= 1) row_max = fmaxf(row_max, __shfl_xor_sync(0xffffffffu, row_max, o));
    float my_logit = 0.f, my_logit_hi = 0.f;
    for (uint32_t r = 0; r < selected; ++r) {
        float best = -INFINITY;
        uint32_t best_id = 0xffffffffu;
#pragma unroll
        for (uint32_t i = 0; i < 16; ++i)
            if (v[i] > best) { best = v[i]; best_id = lane + 32 * i; }   // ascending scan keeps the lowest id on ties
        for (int o = 16; o; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, best_id, o);
            if (ov > best || (ov == best && oi < best_id)) { best = ov; best_id = oi; }
        }
        if ((r & 31u) == lane) { if (r < 32) my_logit = best; else my_logit_hi = best; }
        if (lane == 0) out_ids[r] = best_id;
        if ((best_id & 31u) == lane) {
#pragma unroll
            for (uint32_t i = 0; i < 16; ++i) if ((best_id >> 5) == i) v[i] = -INFINITY;
        }
    }
    const double mx = row_max;
    auto activate = [&](float logit) -> double {
        const double l = logit;
        if (mode == TSP_ROUTER_SOFTMAX) return exp(l - mx);
        return exp(-softplus_f64(-l) + softplus_f64(-mx));
    };
    const double my_act = lane < selected ? activate(my_logit) : 0.0;
    const double my_act_hi = lane + 32 < selected ? activate(my_logit_hi) : 0.0;
    double denominator = my_act + my_act_hi;   // renormalised over the selection: same butterfly order as route_row
    for (int o = 16; o; o >>= 1) denominator += __shfl_xor_sync(0xffffffffu, denominator, o);
    if (!(denominator > 0) || isinf(denominator)) {
        if (lane == 0) raise_error(error, TSP_ERR_NONFINITE);
        denominator = 1.0;
    }
    if (lane < selected) out_w[lane] = static_cast<float>(my_act / denominator);
    if (lane + 32 < selected) out_w[lane + 32] = static_cast<float>(my_act_hi / denominator);
}

__global__ void __launch_bounds__(kRouteWarps * 32)
route_kernel(const float* __restrict__ logits, uint64_t stride_bytes, uint32_t tokens, uint32_t experts,
             uint32_t selected, uint32_t mode, int normalize, uint32_t* __restrict__ ids,
             float* __restrict__ weights, uint32_t* error, float* __restrict__ margins) {
    pdl_launch_dependents();
    pdl_wait();

    extern __shared__ float route_smem[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t token = blockIdx.x * (blockDim.x >> 5) + warp;
    if (token >= tokens) return;
    const float* src = reinterpret_cast<const float*>(reinterpret_cast<const char*>(logits) + token * stride_bytes);
    if (experts <= 512 && normalize && !margins) route_row_regs(src, token, experts, selected, mode, ids, weights, error, lane);
    else route_row(route_smem + warp * experts, src, token, experts, selected, mode, normalize, ids, weights, error, lane, margins);
}

// ---------------------------------------------------------------------------------------------
// permutation: one block per expert compacts, in ascending token order, the routes that name it.
// ---------------------------------------------------------------------------------------------
constexpr int kPermuteThreads = 512;
constexpr uint32_t kPermuteExperts = 2;   // experts per block: a token's ids are read once for all of them

__global__ void __launch_bounds__(kPermuteThreads)
grouped_routes_kernel(const uint32_t* __restrict__ ids, uint32_t tokens, uint32_t experts, uint32_t selected, uint32_t first, int local_only,
                      uint32_t* __restrict__ token_map, uint32_t* __restrict__ counts, uint32_t* error) {
    pdl_launch_dependents();
    pdl_wait();

    __shared__ uint32_t totals[kPermuteExperts][kPermuteThreads / 32];
    const uint32_t e0 = blockIdx.x * kPermuteExperts, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint32_t accumulated[kPermuteExperts];
#pragma unroll
    for (uint32_t q = 0; q < kPermuteExperts; ++q) accumulated[q] = 0;
    for (uint32_t base = 0; base < tokens; base += kPermuteThreads) {
        const uint32_t token = base + tid;
        uint32_t slot[kPermuteExperts], matches[kPermuteExperts];
#pragma unroll
        for (uint32_t q = 0; q < kPermuteExperts; ++q) { slot[q] = 0; matches[q] = 0; }
        if (token < tokens) {
            for (uint32_t i = 0; i < selected; ++i) {
                // ids are global; this launch owns experts [first, first + experts). With local_only, routes to other
                // owners are simply not this rank's business; without it they are an index error.
                const uint32_t id = ids[static_cast<uint64_t>(token) * selected + i] - first;
                if (id >= experts && blockIdx.x == 0 && !local_only) raise_error(error, TSP_ERR_INDEX);
#pragma unroll
                for (uint32_t q = 0; q < kPermuteExperts; ++q)
                    if (id == e0 + q) { slot[q] = i; ++matches[q]; }
            }
        }
        uint32_t prefix[kPermuteExperts];
#pragma unroll
        for (uint32_t q = 0; q < kPermuteExperts; ++q) {
            if (matches[q] > 1) raise_error(error, TSP_ERR_INDEX);
            const uint32_t ballot = __ballot_sync(0xffffffffu, matches[q] == 1);
            prefix[q] = __popc(ballot & ((1u << lane) - 1u));
            if (lane == 0) totals[q][warp] = __popc(ballot);
        }
        __syncthreads();
#pragma unroll
        for (uint32_t q = 0; q < kPermuteExperts; ++q) {
            uint32_t before = 0, chunk = 0;
            for (uint32_t i = 0; i < kPermuteThreads / 32; ++i) { if (i < warp) before += totals[q][i]; chunk += totals[q][i]; }
            if (matches[q] == 1 && e0 + q < experts)
                token_map[static_cast<uint64_t>(e0 + q) * tokens + accumulated[q] + before + prefix[q]] = token * selected + slot[q];
            accumulated[q] += chunk;
        }
        __syncthreads();
    }
    if (tid < kPermuteExperts && e0 + tid < experts) {
        uint32_t c = 0;
#pragma unroll
        for (uint32_t q = 0; q < kPermuteExperts; ++q) if (q == tid) c = accumulated[q];
        counts[e0 + tid] = c;
    }
}

// tasks = {live_tiles, routes, (expert, start) pairs in ascending expert order, 0xffffffff padding}
__global__ void __launch_bounds__(256)
grouped_tasks_kernel(const uint32_t* __restrict__ counts, uint32_t tokens, uint32_t experts, uint32_t selected,
                     uint32_t tile, uint32_t bound, int local_only, uint32_t* __restrict__ tasks, uint32_t* error) {
    pdl_launch_dependents();
    pdl_wait();

    extern __shared__ uint32_t offsets[];  // experts + 1
    const uint32_t tid = threadIdx.x;
    __shared__ uint32_t warp_tiles[8], warp_routes[8];
    // block-wide exclusive scan of tiles per expert, in chunks of 256 experts
    uint32_t carry_tiles = 0, carry_routes = 0;
    for (uint32_t base = 0; base < experts; base += 256) {
        const uint32_t e = base + tid;
        uint32_t c = 0, n = 0;
        if (e < experts) {
            c = counts[e];
            if (c > tokens) raise_error(error, TSP_ERR_INDEX);
            n = (min(c, tokens) + tile - 1) / tile;
        }
        uint32_t incl_n = n, incl_c = c;
        const uint32_t lane = tid & 31, warp = tid >> 5;
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t tn = __shfl_up_sync(0xffffffffu, incl_n, o), tc = __shfl_up_sync(0xffffffffu, incl_c, o);
            if (lane >= static_cast<uint32_t>(o)) { incl_n += tn; incl_c += tc; }
        }
        if (lane == 31) { warp_tiles[warp] = incl_n; warp_routes[warp] = incl_c; }
        __syncthreads();
        uint32_t before_n = 0, total_n = 0, total_c = 0;
        for (uint32_t i = 0; i < 8; ++i) { if (i < warp) before_n += warp_tiles[i]; total_n += warp_tiles[i]; total_c += warp_routes[i]; }
        if (e < experts) offsets[e] = carry_tiles + before_n + incl_n - n;
        carry_tiles += total_n;
        carry_routes += total_c;
        __syncthreads();
    }
    if (tid == 0) {
        offsets[experts] = carry_tiles;
        tasks[0] = min(carry_tiles, bound);
        tasks[1] = carry_routes;
        if (carry_tiles > bound || (!local_only && carry_routes != tokens * selected) || carry_routes > tokens * selected) raise_error(error, TSP_ERR_INDEX);
    }
    for (uint32_t i = tid; i < bound; i += 256) { tasks[2 + 2 * i] = 0xffffffffu; tasks[3 + 2 * i] = 0xffffffffu; }
    __syncthreads();
    for (uint32_t e = tid; e < experts; e += 256) {
        const uint32_t n = (min(counts[e], tokens) + tile - 1) / tile;
        for (uint32_t i = 0; i < n; ++i) {
            const uint32_t at = offsets[e] + i;
            if (at < bound) { tasks[2 + 2 * at] = e; tasks[3 + 2 * at] = i * tile; }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Decode-size prologue of a batch of <= 1024 token rows in TWO launches: (1) routing, one warp per token over as many blocks
// as that takes, with the binary16 -> FP32 copy of the input rows done by the remaining blocks of the same launch (one block
// routing 64 rows alone is bound by its own issue rate: measured 25.7 us); (2) permutation + tile table in one block. The
// tables are the ones the separate kernels above produce, bit for bit: the per-expert token order comes from a bit mask of
// the tokens that name the expert (bit t set = token t routes here), so position = number of lower set bits: no atomics
// decide an order.
// ---------------------------------------------------------------------------------------------
constexpr int kPrologueThreads = 1024;
constexpr int kPrologueRouteWarps = 4;
constexpr uint32_t kPrologueTokens = 1024, kPrologueExperts = 1024;

__global__ void __launch_bounds__(kPrologueRouteWarps * 32)
decode_route_kernel(const float* __restrict__ logits, uint64_t logits_stride, uint32_t tokens, uint32_t experts, uint32_t selected,
                    uint32_t mode, int normalize, uint32_t route_blocks, uint32_t* __restrict__ ids, float* __restrict__ weights,
                    const __half* __restrict__ x16, uint64_t x16_stride, float* __restrict__ x32, uint64_t x32_stride, uint32_t channels,
                    uint32_t* error) {
    pdl_launch_dependents();
    pdl_wait();
    if (blockIdx.x >= route_blocks) {   // the conversion blocks: binary16 rows -> FP32 rows (exact)
        const uint32_t per_row = channels / 4;   // four values per thread step
        const uint32_t nconv = gridDim.x - route_blocks;
        for (uint32_t i = (blockIdx.x - route_blocks) * blockDim.x + threadIdx.x; i < tokens * per_row; i += nconv * blockDim.x) {
            const uint32_t row = i / per_row, c4 = i - row * per_row;
            const uint2 h = *reinterpret_cast<const uint2*>(reinterpret_cast<const char*>(x16) + row * x16_stride + c4 * 8ull);
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&h.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&h.y));
            *reinterpret_cast<float4*>(reinterpret_cast<char*>(x32) + row * x32_stride + c4 * 16ull) = make_float4(a.x, a.y, b.x, b.y);
        }
        return;
    }
    extern __shared__ float pro_smem[];          // [warps][experts] routing rows of the shared-memory form
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t t = blockIdx.x * kPrologueRouteWarps + warp;
    if (t >= tokens) return;
    const float* row = reinterpret_cast<const float*>(reinterpret_cast<const char*>(logits) + t * logits_stride);
    if (experts <= 512 && normalize) route_row_regs(row, t, experts, selected, mode, ids, weights, error, lane);
    else route_row(pro_smem + warp * experts, row, t, experts, selected, mode, normalize, ids, weights, error, lane);
}

// Permutation + tile table of up to 1024 token rows in ONE block: a mask of the rows that name each expert (`words` 32-bit words per
// expert in shared memory), positions = number of lower set bits. ids are global; this launch owns experts [first, first + experts);
// with local_only, routes to other owners are skipped, without it they are an index error.
__global__ void __launch_bounds__(kPrologueThreads)
tables_kernel(const uint32_t* __restrict__ ids, uint32_t tokens, uint32_t experts, uint32_t selected, uint32_t tile, uint32_t first, int local_only,
              uint32_t words, uint32_t* __restrict__ token_map, uint32_t* __restrict__ counts, uint32_t* __restrict__ tasks, uint32_t* error) {
    pdl_launch_dependents();
    extern __shared__ uint32_t tables_mask[];   // [experts][words]
    __shared__ uint32_t warp_tiles[32], warp_routes[32];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
    for (uint32_t i = tid; i < experts * words; i += blockDim.x) tables_mask[i] = 0u;
    const uint32_t routes = tokens * selected;
    const uint32_t bound = routes / tile + experts;
    pdl_wait();   // the ids come from the previous launch; everything above touched shared memory only
    __syncthreads();
    for (uint32_t i = tid; i < routes; i += blockDim.x) {
        const uint32_t t = i / selected, e = ids[i] - first;
        if (e >= experts) { if (!local_only) raise_error(error, TSP_ERR_INDEX); continue; }
        const uint32_t bit = 1u << (t & 31u);
        if (atomicOr(&tables_mask[e * words + (t >> 5)], bit) & bit) raise_error(error, TSP_ERR_INDEX);   // an expert named twice by one token
    }
    for (uint32_t i = tid; i < bound; i += blockDim.x) { tasks[2 + 2 * i] = 0xffffffffu; tasks[3 + 2 * i] = 0xffffffffu; }
    __syncthreads();
    for (uint32_t i = tid; i < routes; i += blockDim.x) {
        const uint32_t t = i / selected, e = ids[i] - first;
        if (e >= experts) continue;
        const uint32_t* m = tables_mask + e * words;
        uint32_t j = __popc(m[t >> 5] & ((1u << (t & 31u)) - 1u));
        for (uint32_t w = 0; w < (t >> 5); ++w) j += __popc(m[w]);
        token_map[static_cast<uint64_t>(e) * tokens + j] = i;
    }
    // tile table: exclusive scan of tiles per expert over the block (experts <= blockDim.x)
    uint32_t c = 0, n = 0;
    if (tid < experts) {
        for (uint32_t w = 0; w < words; ++w) c += __popc(tables_mask[tid * words + w]);
        n = (c + tile - 1) / tile;
        counts[tid] = c;
    }
    uint32_t incl_n = n, incl_c = c;
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t tn = __shfl_up_sync(0xffffffffu, incl_n, o), tc = __shfl_up_sync(0xffffffffu, incl_c, o);
        if (lane >= static_cast<uint32_t>(o)) { incl_n += tn; incl_c += tc; }
    }
    if (lane == 31) { warp_tiles[warp] = incl_n; warp_routes[warp] = incl_c; }
    __syncthreads();   // also orders the padding of the tile table above before the entries below
    uint32_t before = 0, total_n = 0, total_c = 0;
    for (uint32_t i = 0; i < nwarps; ++i) { if (i < warp) before += warp_tiles[i]; total_n += warp_tiles[i]; total_c += warp_routes[i]; }
    if (tid == 0) {
        tasks[0] = min(total_n, bound);
        tasks[1] = total_c;
        if (total_n > bound || (!local_only && total_c != routes) || total_c > routes) raise_error(error, TSP_ERR_INDEX);
    }
    if (tid < experts) {
        const uint32_t at0 = before + incl_n - n;
        for (uint32_t i = 0; i < n; ++i) {
            const uint32_t at = at0 + i;
            if (at < bound) { tasks[2 + 2 * at] = tid; tasks[3 + 2 * at] = i * tile; }
        }
    }
}

// The one-block form covers up to 1024 rows and experts whose masks fit 96 KB of shared memory.
static bool tables_fit(uint32_t tokens, uint32_t experts) {
    return tokens >= 1 && tokens <= 1024 && experts <= static_cast<uint32_t>(kPrologueThreads) && static_cast<uint64_t>(experts) * ((tokens + 31) / 32) * 4 <= 96 * 1024;
}
static int launch_tables(const uint32_t* ids, uint32_t tokens, uint32_t experts, uint32_t selected, uint32_t tile, uint32_t first, int local_only,
                         uint32_t* token_map, uint32_t* counts, uint32_t* tasks, uint32_t* error, cudaStream_t st) {
    const uint32_t words = (tokens + 31) / 32;
    const size_t smem = static_cast<size_t>(experts) * words * 4;
    static thread_local SmemAttrCache configured;
    TSP_CUDA(ensure_dynamic_smem(tables_kernel, configured, smem));
    TSP_CUDA(launch_pdl(tables_kernel, dim3(1), dim3(kPrologueThreads), smem, st, ids, tokens, experts, selected, tile, first, local_only, words, token_map, counts,
                        tasks, error));
    return TSP_OK;
}

// Returns 1 when the batch does not fit the short prologue (the caller then issues the separate launches).
int launch_decode_prologue(const float* logits, uint64_t logits_stride, uint32_t tokens, uint32_t experts, uint32_t selected, uint32_t mode,
                           int normalize, uint32_t tile, uint32_t* ids, float* weights, uint32_t* token_map, uint32_t* counts, uint32_t* tasks,
                           const void* x16, uint64_t x16_stride, float* x32, uint64_t x32_stride, uint32_t channels, uint32_t* error, cudaStream_t st) {
    if (tokens > kPrologueTokens || experts > kPrologueExperts || !tables_fit(tokens, experts)) return 1;
    if (x16 && (channels % 4 || x16_stride % 8 || x32_stride % 16 || reinterpret_cast<uintptr_t>(x16) % 8 || reinterpret_cast<uintptr_t>(x32) % 16)) return 1;
    const size_t smem = (experts <= 512 && normalize) ? 0 : static_cast<size_t>(kPrologueRouteWarps) * experts * sizeof(float);
    static thread_local SmemAttrCache configured;
    TSP_CUDA(ensure_dynamic_smem(decode_route_kernel, configured, smem));
    const uint32_t route_blocks = (tokens + kPrologueRouteWarps - 1) / kPrologueRouteWarps;
    // conversion blocks: enough to cover the rows in two passes
    const uint32_t conv = x16 ? min(128u, (tokens * (channels / 4) + 2 * kPrologueRouteWarps * 32 - 1) / (2 * kPrologueRouteWarps * 32)) : 0u;
    TSP_CUDA(launch_pdl(decode_route_kernel, dim3(route_blocks + conv), dim3(kPrologueRouteWarps * 32), smem, st, logits, logits_stride, tokens, experts,
                        selected, mode, normalize, route_blocks, ids, weights, static_cast<const __half*>(x16), x16_stride, x32, x32_stride, channels, error));
    if (int rc = launch_tables(ids, tokens, experts, selected, tile, 0, 0, token_map, counts, tasks, error, st)) return rc;
    TSP_CUDA(cudaGetLastError());
    return TSP_OK;
}

// ---------------------------------------------------------------------------------------------
// combine: one block per token. Optional shared-router dot (FP32 tree sum), then the mixture in
// route-rank order starting from the gated shared term (routing.cpp:49-58).
// ---------------------------------------------------------------------------------------------
constexpr int kCombineThreads = 256;

// R16: the route rows are binary16 (the prefill path keeps them so); X16: the input rows of the shared-router dot are binary16.
template <bool R16, bool X16>
__global__ void __launch_bounds__(kCombineThreads)
combine_kernel(const void* __restrict__ routed, uint64_t routed_stride, const float* __restrict__ weights,
               const float* __restrict__ shared, uint64_t shared_stride, const float* __restrict__ shared_router,
               const void* __restrict__ x, uint64_t x_stride, float* shared_logit, uint32_t channels,
               uint32_t selected, float* __restrict__ out, uint64_t out_stride, __half* __restrict__ out16,
               uint64_t out16_stride, int vec4, uint32_t* error) {
    pdl_launch_dependents();
    pdl_wait();

    __shared__ float partial[kCombineThreads / 32];
    __shared__ float w_s[64];
    __shared__ float gate_s;
    const uint32_t token = blockIdx.x, tid = threadIdx.x;
    if (tid < selected) w_s[tid] = weights[static_cast<uint64_t>(token) * selected + tid];
    float gate = 1.f;
    if (shared_router) {
        const char* xr = reinterpret_cast<const char*>(x) + token * x_stride;
        float acc = 0.f;
        for (uint32_t c = tid; c < channels; c += kCombineThreads)
            acc = fmaf(shared_router[c], X16 ? __half2float(reinterpret_cast<const __half*>(xr)[c]) : reinterpret_cast<const float*>(xr)[c], acc);
        for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if ((tid & 31) == 0) partial[tid >> 5] = acc;
        __syncthreads();
        if (tid == 0) {
            float s = 0.f;
            for (int i = 0; i < kCombineThreads / 32; ++i) s += partial[i];
            if (!finite_f32(s)) raise_error(error, TSP_ERR_NONFINITE);
            if (shared_logit && blockIdx.y == 0) shared_logit[token] = s;
            gate_s = stable_sigmoid(s);
        }
        __syncthreads();
        gate = gate_s;
    } else {
        if (shared_logit) gate = stable_sigmoid(shared_logit[token]);
        __syncthreads();
    }
    // shared == nullptr: no shared term (the rows are partial sums that another launch finishes)
    const float* sh = shared ? reinterpret_cast<const float*>(reinterpret_cast<const char*>(shared) + token * shared_stride) : nullptr;
    float* o = reinterpret_cast<float*>(reinterpret_cast<char*>(out) + token * out_stride);
    bool bad = false;
    // gridDim.y slices of the row per token, so that a small batch still fills the machine while a large one does not repeat
    // the gate's dot product more often than needed; four channels per thread (rows are 16-byte aligned)
    const uint32_t per_slice = ((channels + gridDim.y - 1) / gridDim.y + 3u) & ~3u;
    const uint32_t c_end = min(channels, (blockIdx.y + 1) * per_slice);
    const char* y0 = reinterpret_cast<const char*>(routed) + static_cast<uint64_t>(token) * selected * routed_stride;
    if (R16 && vec4 == 2 && (channels & 7u) == 0 && gridDim.y == 1) {   // vec4 == 2: every row of every buffer starts on a 16-byte boundary
        // binary16 route rows (prefill): eight channels per thread step, one 16-byte load per route row, five rows in flight
        for (uint32_t c = tid * 8; c < channels; c += kCombineThreads * 8) {
            float v[8];
            if (sh) {
                const float4 a = *reinterpret_cast<const float4*>(sh + c), b = *reinterpret_cast<const float4*>(sh + c + 4);
                v[0] = gate * a.x; v[1] = gate * a.y; v[2] = gate * a.z; v[3] = gate * a.w; v[4] = gate * b.x; v[5] = gate * b.y; v[6] = gate * b.z; v[7] = gate * b.w;
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = 0.f;
            }
            for (uint32_t r0 = 0; r0 < selected; r0 += 5) {
                uint4 y[5];
#pragma unroll
                for (uint32_t i = 0; i < 5; ++i) y[i] = *reinterpret_cast<const uint4*>(y0 + min(r0 + i, selected - 1) * routed_stride + c * 2ull);
#pragma unroll
                for (uint32_t i = 0; i < 5; ++i) {
                    const float wr = r0 + i < selected ? w_s[r0 + i] : 0.f;
                    if (wr != 0.f) {
                        const uint32_t w4[4] = {y[i].x, y[i].y, y[i].z, y[i].w};
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w4[q]));
                            v[2 * q] = fmaf(wr, f.x, v[2 * q]); v[2 * q + 1] = fmaf(wr, f.y, v[2 * q + 1]);
                        }
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) bad |= !finite_f32(v[i]);
            if (out) { *reinterpret_cast<float4*>(o + c) = make_float4(v[0], v[1], v[2], v[3]); *reinterpret_cast<float4*>(o + c + 4) = make_float4(v[4], v[5], v[6], v[7]); }
            if (out16) {
                uint32_t h[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) { const __half2 t2 = __floats2half2_rn(v[2 * q], v[2 * q + 1]); h[q] = *reinterpret_cast<const uint32_t*>(&t2); }
                *reinterpret_cast<uint4*>(reinterpret_cast<char*>(out16) + token * out16_stride + c * 2ull) = make_uint4(h[0], h[1], h[2], h[3]);
            }
        }
        if (bad) raise_error(error, TSP_ERR_NONFINITE);
        return;
    }
    for (uint32_t c = blockIdx.y * per_slice + tid * 4; c < c_end; c += kCombineThreads * 4) {
        if (vec4 && c + 4 <= c_end) {
            const float4 s4 = sh ? *reinterpret_cast<const float4*>(sh + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            float v[4] = {gate * s4.x, gate * s4.y, gate * s4.z, gate * s4.w};
            // A zero weight marks a route that is not present in `routed` (expert parallelism): its row is still inside the
            // buffer, so it is loaded like the others (four rows in flight) and only the sum skips it.
            for (uint32_t r0 = 0; r0 < selected; r0 += 4) {
                float4 y[4];
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i) {
                    const uint32_t r = min(r0 + i, selected - 1);
                    if (R16) {
                        const uint2 h = *reinterpret_cast<const uint2*>(y0 + r * routed_stride + c * 2ull);
                        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&h.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&h.y));
                        y[i] = make_float4(a.x, a.y, b.x, b.y);
                    } else {
                        y[i] = *reinterpret_cast<const float4*>(y0 + r * routed_stride + c * 4ull);
                    }
                }
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i) {
                    const float wr = r0 + i < selected ? w_s[r0 + i] : 0.f;
                    if (wr != 0.f) { v[0] = fmaf(wr, y[i].x, v[0]); v[1] = fmaf(wr, y[i].y, v[1]); v[2] = fmaf(wr, y[i].z, v[2]); v[3] = fmaf(wr, y[i].w, v[3]); }
                }
            }
            bad |= !finite_f32(v[0]) | !finite_f32(v[1]) | !finite_f32(v[2]) | !finite_f32(v[3]);
            if (out) *reinterpret_cast<float4*>(o + c) = make_float4(v[0], v[1], v[2], v[3]);
            if (out16) {
                const __half2 h0 = __floats2half2_rn(v[0], v[1]), h1 = __floats2half2_rn(v[2], v[3]);
                *reinterpret_cast<uint2*>(reinterpret_cast<char*>(out16) + token * out16_stride + c * 2ull) =
                    make_uint2(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
            }
        } else {
            for (uint32_t cc = c; cc < min(c + 4, c_end); ++cc) {   // a row tail shorter than four channels, or rows that are not 16-byte aligned
                float v = sh ? gate * sh[cc] : 0.f;
                for (uint32_t r = 0; r < selected; ++r)
                    if (w_s[r] != 0.f) {
                        const char* yr = y0 + r * routed_stride;
                        v = fmaf(w_s[r], R16 ? __half2float(reinterpret_cast<const __half*>(yr)[cc]) : reinterpret_cast<const float*>(yr)[cc], v);
                    }
                bad |= !finite_f32(v);
                if (out) o[cc] = v;
                if (out16) reinterpret_cast<__half*>(reinterpret_cast<char*>(out16) + token * out16_stride)[cc] = __float2half_rn(v);
            }
        }
    }
    if (bad) raise_error(error, TSP_ERR_NONFINITE);
}

// ---------------------------------------------------------------------------------------------
// F32 matrix-vector product for the router projections: one warp per (matrix row, token), FP32 FMA + tree sum.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gemv_f32_kernel(const float* __restrict__ w, uint32_t rows, uint32_t cols, const float* __restrict__ x, uint64_t x_stride, uint32_t tokens,
                float* __restrict__ out, uint64_t out_stride, uint32_t* error) {
    pdl_launch_dependents();
    pdl_wait();

    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= rows * tokens) return;
    const uint32_t token = warp / rows, row = warp % rows;
    const float* wr = w + static_cast<uint64_t>(row) * cols;
    const float* xr = reinterpret_cast<const float*>(reinterpret_cast<const char*>(x) + token * x_stride);
    float acc = 0.f;
    for (uint32_t c = lane; c < cols; c += 32) acc = fmaf(wr[c], xr[c], acc);
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
        if (!finite_f32(acc)) raise_error(error, TSP_ERR_NONFINITE);
        reinterpret_cast<float*>(reinterpret_cast<char*>(out) + token * out_stride)[row] = acc;
    }
}

// ---------------------------------------------------------------------------------------------
// F32 router projection for batches: logits[t][e] = sum_c W[e][c] * x[t][c] as a register-tiled FP32 GEMM (FP32 FMA only: the
// ids chosen from these logits must follow the reference's double-precision logits, so no reduced-precision tensor path).
// W is read once per tile of 64 token rows. Every output is one FMA chain in ascending c, i.e. the plain sequential FP32 dot
// product. An optional extra row `extra` (the shared-router vector) is projected in the same pass into `extra_out[t]`.
// ---------------------------------------------------------------------------------------------
constexpr int kRgM = 64, kRgN = 128, kRgK = 16, kRgThreads = 256;

__global__ void __launch_bounds__(kRgThreads)
router_gemm_kernel(const float* __restrict__ w, uint32_t rows, uint32_t cols, const float* __restrict__ extra, const float* __restrict__ x,
                   uint64_t x_stride, uint32_t tokens, float* __restrict__ out, uint64_t out_stride, float* __restrict__ extra_out, uint32_t* error) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float xs[kRgK][kRgM + 4];
    __shared__ float ws[kRgK][kRgN + 4];
    const uint32_t tid = threadIdx.x;
    const uint32_t t0 = blockIdx.y * kRgM, r0 = blockIdx.x * kRgN;
    const uint32_t all_rows = rows + (extra ? 1u : 0u);
    // thread -> 4 token rows x 8 matrix rows of the tile
    const uint32_t tm = (tid >> 4) * 4, tn = (tid & 15u) * 8;
    float acc[4][8];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
    // loaders: x tile = 64 rows x 16 columns = 256 float4 (one per thread); w tile = 128 x 16 = 512 float4 (two per thread)
    const uint32_t lx_row = tid >> 2, lx_c4 = (tid & 3u) * 4;
    for (uint32_t k0 = 0; k0 < cols; k0 += kRgK) {
        {
            const uint32_t t = t0 + lx_row, c = k0 + lx_c4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t < tokens) {
                const float* src = reinterpret_cast<const float*>(reinterpret_cast<const char*>(x) + t * x_stride) + c;
                if (c + 4 <= cols && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) v = *reinterpret_cast<const float4*>(src);
                else { if (c < cols) v.x = src[0]; if (c + 1 < cols) v.y = src[1]; if (c + 2 < cols) v.z = src[2]; if (c + 3 < cols) v.w = src[3]; }
            }
            xs[lx_c4][lx_row] = v.x; xs[lx_c4 + 1][lx_row] = v.y; xs[lx_c4 + 2][lx_row] = v.z; xs[lx_c4 + 3][lx_row] = v.w;
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t lr = (tid >> 2) + h * 64, r = r0 + lr, c = k0 + lx_c4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (r < all_rows) {
                const float* src = (r < rows ? w + static_cast<uint64_t>(r) * cols : extra) + c;
                if (c + 4 <= cols && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) v = *reinterpret_cast<const float4*>(src);
                else { if (c < cols) v.x = src[0]; if (c + 1 < cols) v.y = src[1]; if (c + 2 < cols) v.z = src[2]; if (c + 3 < cols) v.w = src[3]; }
            }
            ws[lx_c4][lr] = v.x; ws[lx_c4 + 1][lr] = v.y; ws[lx_c4 + 2][lr] = v.z; ws[lx_c4 + 3][lr] = v.w;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kRgK; ++k) {
            const float4 a = *reinterpret_cast<const float4*>(&xs[k][tm]);
            const float4 b0 = *reinterpret_cast<const float4*>(&ws[k][tn]), b1 = *reinterpret_cast<const float4*>(&ws[k][tn + 4]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(bv[j], av[i], acc[i][j]);
        }
        __syncthreads();
    }
    bool bad = false;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t t = t0 + tm + i;
        if (t >= tokens) continue;
        float* orow = reinterpret_cast<float*>(reinterpret_cast<char*>(out) + t * out_stride);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t r = r0 + tn + j;
            if (r < rows) { bad |= !finite_f32(acc[i][j]); orow[r] = acc[i][j]; }
            else if (r == rows && extra) { bad |= !finite_f32(acc[i][j]); extra_out[t] = acc[i][j]; }
        }
    }
    if (bad) raise_error(error, TSP_ERR_NONFINITE);
}

// The same product for large batches: K steps of 16 double-buffered in shared memory, every shared-memory load 16 bytes and
// conflict-free, FP32 FMA in ascending K order per output. Requires cols % 16 == 0 and 16-byte aligned rows; edge tiles are
// predicated. (The 64 x 128 kernel above, no double buffering, ran at 15 TFLOP/s on 4096 x 512 x 2048: 0.574 ms.)
constexpr int kSgT = 128, kSgK = 16, kSgThreads = 256;

// One block: 128 token rows x 64 matrix rows, 8 x 4 outputs per thread, two blocks per SM. Measured on 4096 x 512 x 2048
// (ms): this form 0.278; 128 x 128 tiles with 8 x 8 outputs (one block per SM, 128 blocks) 0.402; packed FP32 FMAs 0.280
// (the kernel is not bound by issue slots); a warp-broadcast mapping with 16 x 4 outputs 0.415.
__global__ void __launch_bounds__(kSgThreads, 2)
router_sgemm_kernel(const float* __restrict__ w, uint32_t rows, uint32_t cols, const float* __restrict__ x, uint64_t x_stride, uint32_t tokens,
                    float* __restrict__ out, uint64_t out_stride, uint32_t* error) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int TN = 64;
    __shared__ __align__(16) float xs[2][kSgK][kSgT];
    __shared__ __align__(16) float ws[2][kSgK][TN];
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t t0 = blockIdx.y * kSgT, r0 = blockIdx.x * TN;
    // loaders: a warp takes 32 consecutive rows of a tile and one 4-wide K group; stores to [k][row] are then bank-conflict-free
    const uint32_t l_row = lane + 32 * (warp & 3u), l_k = 4 * (warp >> 2);   // x: K groups l_k and l_k + 8
    const uint32_t w_row = lane + 32 * (warp & 1u), w_k = 4 * (warp >> 1);   // w: 64 rows, one K group per warp
    const float* xsrc = reinterpret_cast<const float*>(reinterpret_cast<const char*>(x) + static_cast<uint64_t>(min(t0 + l_row, tokens - 1)) * x_stride);
    const float* wsrc = w + static_cast<uint64_t>(min(r0 + w_row, rows - 1)) * cols;
    // outputs: token rows ty*4 + {0..3} and 64 + ty*4 + {0..3}, matrix rows tx*4 + {0..3}
    const uint32_t ty = tid >> 4, tx = tid & 15u;
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    float4 gx[2], gw;
    auto fetch = [&](uint32_t k0) {
        gx[0] = *reinterpret_cast<const float4*>(xsrc + k0 + l_k); gx[1] = *reinterpret_cast<const float4*>(xsrc + k0 + l_k + 8);
        gw = *reinterpret_cast<const float4*>(wsrc + k0 + w_k);
    };
    auto stash = [&](uint32_t b) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t k = l_k + 8 * h;
            xs[b][k][l_row] = gx[h].x; xs[b][k + 1][l_row] = gx[h].y; xs[b][k + 2][l_row] = gx[h].z; xs[b][k + 3][l_row] = gx[h].w;
        }
        ws[b][w_k][w_row] = gw.x; ws[b][w_k + 1][w_row] = gw.y; ws[b][w_k + 2][w_row] = gw.z; ws[b][w_k + 3][w_row] = gw.w;
    };
    fetch(0);
    stash(0);
    __syncthreads();
    uint32_t buf = 0;
    for (uint32_t k0 = 0; k0 < cols; k0 += kSgK) {
        const bool more = k0 + kSgK < cols;
        if (more) fetch(k0 + kSgK);
#pragma unroll
        for (int k = 0; k < kSgK; ++k) {
            const float4 a0 = *reinterpret_cast<const float4*>(&xs[buf][k][ty * 4]), a1 = *reinterpret_cast<const float4*>(&xs[buf][k][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&ws[buf][k][tx * 4]);
            const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w}, bv[4] = {b0.x, b0.y, b0.z, b0.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(bv[j], av[i], acc[i][j]);
        }
        if (more) stash(buf ^ 1u);
        __syncthreads();
        buf ^= 1u;
    }
    bool bad = false;
    const uint32_t r = r0 + tx * 4;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t t = t0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (t >= tokens) continue;
        float* orow = reinterpret_cast<float*>(reinterpret_cast<char*>(out) + t * out_stride);
#pragma unroll
        for (int j = 0; j < 4; ++j) bad |= !finite_f32(acc[i][j]) && r + j < rows;
        if (r + 4 <= rows && (reinterpret_cast<uintptr_t>(orow + r) & 15u) == 0) *reinterpret_cast<float4*>(orow + r) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        else
            for (int j = 0; j < 4; ++j) if (r + j < rows) orow[r + j] = acc[i][j];
    }
    if (bad) raise_error(error, TSP_ERR_NONFINITE);
}

int launch_gemv_f32(const float* w, uint32_t rows, uint32_t cols, const float* extra, const float* x, uint64_t x_stride, uint32_t tokens, float* out,
                    uint64_t out_stride, float* extra_out, uint32_t* error, cudaStream_t st) {
    if (tokens >= 256 && rows >= 64 && cols % kSgK == 0 && (reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x) | x_stride) % 16 == 0) {
        // large batches: full 128 x 128 tiles; the extra row (one dot product per token) takes its own small launch
        const dim3 grid((rows + 63) / 64, (tokens + kSgT - 1) / kSgT);
        TSP_CUDA(launch_pdl(router_sgemm_kernel, grid, dim3(kSgThreads), 0, st, w, rows, cols, x, x_stride, tokens, out, out_stride, error));
        if (extra) TSP_CUDA(launch_pdl(gemv_f32_kernel, dim3(static_cast<unsigned>((tokens + 7) / 8)), dim3(256), 0, st, extra, 1u, cols, x, x_stride, tokens, extra_out, sizeof(float), error));
        return TSP_OK;
    }
    if (tokens >= 32) {   // batches: W is read once per 64 token rows
        const dim3 grid((rows + (extra ? 1 : 0) + kRgN - 1) / kRgN, (tokens + kRgM - 1) / kRgM);
        TSP_CUDA(launch_pdl(router_gemm_kernel, grid, dim3(kRgThreads), 0, st, w, rows, cols, extra, x, x_stride, tokens, out, out_stride, extra_out, error));
        return TSP_OK;
    }
    const uint64_t warps = static_cast<uint64_t>(rows) * tokens;
    TSP_CUDA(launch_pdl(gemv_f32_kernel, dim3(static_cast<unsigned>((warps + 7) / 8)), dim3(256), 0, st, w, rows, cols, x, x_stride, tokens, out, out_stride, error));
    if (extra) TSP_CUDA(launch_pdl(gemv_f32_kernel, dim3(static_cast<unsigned>((tokens + 7) / 8)), dim3(256), 0, st, extra, 1u, cols, x, x_stride, tokens, extra_out, sizeof(float), error));
    return TSP_OK;
}

__global__ void rows_f16_to_f32_kernel(const __half* __restrict__ in, uint64_t in_stride, float* __restrict__ out,
                                       uint64_t out_stride, uint32_t rows, uint32_t cols) {
    pdl_launch_dependents();
    pdl_wait();

    const uint32_t row = blockIdx.y;
    const __half* src = reinterpret_cast<const __half*>(reinterpret_cast<const char*>(in) + row * in_stride);
    float* dst = reinterpret_cast<float*>(reinterpret_cast<char*>(out) + row * out_stride);
    for (uint32_t c = blockIdx.x * blockDim.x + threadIdx.x; c < cols; c += gridDim.x * blockDim.x) dst[c] = __half2float(src[c]);
}

// ---------------------------------------------------------------------------------------------
// dequantise test hook: FP32 fmaf(d*sc, q, -(dmin*mn)) is the exactly rounded reference value
// because d*sc, (d*sc)*q and dmin*mn are exact in FP32 (at most 21 significant bits).
// ---------------------------------------------------------------------------------------------
__global__ void dequant_q4k_kernel(const uint8_t* __restrict__ expert, uint32_t layout, uint64_t total_blocks,
                                   float* __restrict__ out, uint32_t* error) {
    const uint64_t blk = blockIdx.x;
    const uint32_t i = threadIdx.x;  // 0..255
    const uint32_t g = i >> 5;
    uint32_t dbits, mbits, sc, mn, q;
    if (layout == TSP_LAYOUT_GGUF) {
        const uint8_t* b = expert + blk * 144;
        dbits = b[0] | (b[1] << 8);
        mbits = b[2] | (b[3] << 8);
        if (g < 4) { sc = b[4 + g] & 63u; mn = b[8 + g] & 63u; }
        else { sc = (b[12 + g - 4] & 15u) | ((b[4 + g - 4] >> 6) << 4); mn = (b[12 + g - 4] >> 4) | ((b[8 + g - 4] >> 6) << 4); }
        q = (b[16 + (i >> 6) * 32 + (i & 31)] >> (4 * ((i >> 5) & 1))) & 15u;
    } else {
        const uint8_t* qs = expert + blk * 128;
        const uint8_t* sm = expert + total_blocks * 128 + blk * 16;
        const uint8_t* dm = expert + total_blocks * 144 + blk * 4;
        dbits = dm[0] | (dm[1] << 8);
        mbits = dm[2] | (dm[3] << 8);
        sc = sm[g]; mn = sm[8 + g];
        if ((sc | mn) & 0xc0u) raise_error(error, TSP_ERR_INDEX);
        q = (qs[(i >> 6) * 32 + (i & 31)] >> (4 * ((i >> 5) & 1))) & 15u;
    }
    const float d = half_bits_to_float(dbits), dmin = half_bits_to_float(mbits);
    const float v = fmaf(d * static_cast<float>(sc), static_cast<float>(q), -(dmin * static_cast<float>(mn)));
    if (!finite_f32(v) || !finite_f32(d) || !finite_f32(dmin)) raise_error(error, TSP_ERR_NONFINITE);
    out[blk * 256 + i] = v;
}

__global__ void dequant_q8_kernel(const uint8_t* __restrict__ expert, uint32_t layout, uint64_t total_blocks,
                                  float* __restrict__ out, uint32_t* error) {
    const uint64_t blk = static_cast<uint64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (blk >= total_blocks) return;
    const uint32_t i = threadIdx.x & 31;
    uint32_t dbits;
    int q;
    if (layout == TSP_LAYOUT_GGUF) {
        const uint8_t* b = expert + blk * 34;
        dbits = b[0] | (b[1] << 8);
        q = static_cast<int8_t>(b[2 + i]);
    } else {
        const uint8_t* dm = expert + total_blocks * 32 + blk * 2;
        dbits = dm[0] | (dm[1] << 8);
        q = static_cast<int8_t>(expert[blk * 32 + i]);
    }
    const float d = half_bits_to_float(dbits);
    const float v = d * static_cast<float>(q);
    if (!finite_f32(v)) raise_error(error, TSP_ERR_NONFINITE);
    out[blk * 32 + i] = v;
}

// ---------------------------------------------------------------------------------------------
// host launchers (called by the C ABI layer in tsp_api.cu after validation)
// ---------------------------------------------------------------------------------------------
int launch_route(const float* logits, uint64_t stride, uint32_t tokens, uint32_t experts, uint32_t selected,
                 uint32_t mode, int normalize, uint32_t* ids, float* weights, uint32_t* error, cudaStream_t st, float* margins) {
    const uint32_t warps = experts > 3072 ? 2 : kRouteWarps;
    const uint32_t blocks = (tokens + warps - 1) / warps;
    TSP_CUDA(launch_pdl(route_kernel, dim3(blocks), dim3(warps * 32), warps * experts * sizeof(float), st, logits, stride, tokens, experts, selected, mode, normalize, ids, weights, error, margins));
    TSP_CUDA(cudaGetLastError());
    return TSP_OK;
}

int launch_permute(const uint32_t* ids, uint32_t tokens, uint32_t experts, uint32_t selected, uint32_t tile, uint32_t first, int local_only,
                   uint32_t* token_map, uint32_t* counts, uint32_t* tasks, uint32_t* error, cudaStream_t st) {
    if (tables_fit(tokens, experts)) return launch_tables(ids, tokens, experts, selected, tile, first, local_only, token_map, counts, tasks, error, st);
    TSP_CUDA(launch_pdl(grouped_routes_kernel, dim3((experts + kPermuteExperts - 1) / kPermuteExperts), dim3(kPermuteThreads), 0, st, ids, tokens, experts, selected, first, local_only, token_map, counts, error));
    TSP_CUDA(cudaGetLastError());
    const uint32_t bound = static_cast<uint32_t>((static_cast<uint64_t>(tokens) * selected) / tile + experts);
    TSP_CUDA(launch_pdl(grouped_tasks_kernel, dim3(1), dim3(256), (experts + 1) * sizeof(uint32_t), st, counts, tokens, experts, selected, tile, bound, local_only, tasks, error));
    TSP_CUDA(cudaGetLastError());
    return TSP_OK;
}

int launch_combine(const void* routed, uint64_t routed_stride, uint32_t routed_f16, const float* weights, const float* shared,
                   uint64_t shared_stride, const float* shared_router, const void* x, uint64_t x_stride, uint32_t x_f16,
                   float* shared_logit, uint32_t tokens, uint32_t channels, uint32_t selected, float* out,
                   uint64_t out_stride, void* out16, uint64_t out16_stride, uint32_t* error, cudaStream_t st) {
    // about four CTAs per SM in total: 8 slices of a 2048-wide row at 64 tokens, one slice from a few hundred tokens on
    uint32_t slices = (channels + kCombineThreads - 1) / kCombineThreads;
    const uint32_t want = (4u * 148u + tokens - 1) / tokens;
    if (slices > want) slices = want;
    auto a16 = [](const void* p, uint64_t stride) { return (reinterpret_cast<uintptr_t>(p) | stride) % 16 == 0; };
    const int vec4 = (routed_f16 ? (reinterpret_cast<uintptr_t>(routed) | routed_stride) % 8 == 0 : a16(routed, routed_stride)) && (!shared || a16(shared, shared_stride)) &&
                     (!out || a16(out, out_stride)) && (!out16 || (reinterpret_cast<uintptr_t>(out16) | out16_stride) % 8 == 0);
    const int vec8 = vec4 && routed_f16 && a16(routed, routed_stride) && (!out16 || a16(out16, out16_stride));
    const dim3 grid(tokens, slices), block(kCombineThreads);
#define TSP_COMBINE(R, X) TSP_CUDA(launch_pdl(combine_kernel<R, X>, grid, block, 0, st, routed, routed_stride, weights, shared, shared_stride, shared_router, \
                                              x, x_stride, shared_logit, channels, selected, out, out_stride, static_cast<__half*>(out16), out16_stride, vec8 ? 2 : vec4, error))
    if (routed_f16) { if (x_f16) TSP_COMBINE(true, true); else TSP_COMBINE(true, false); }
    else { if (x_f16) TSP_COMBINE(false, true); else TSP_COMBINE(false, false); }
#undef TSP_COMBINE
    TSP_CUDA(cudaGetLastError());
    return TSP_OK;
}

// One thread waits on a barrier that nothing ever arrives on, with a small poll limit: the wait gives up, the kernel reports
// TSP_ERR_TIMEOUT through the error word and returns normally. This is the path every bounded wait of the library takes when
// an arrival is lost; it is exercised here without making any real pipeline misbehave.
__global__ void bounded_wait_selftest_kernel(uint32_t polls, uint32_t* error) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
    __syncthreads();
    if (threadIdx.x == 0 && !mbar_wait(&bar, 0, polls)) raise_error(error, TSP_ERR_TIMEOUT);
}

int launch_bounded_wait_selftest(uint32_t polls, uint32_t* error, cudaStream_t st) {
    bounded_wait_selftest_kernel<<<1, 32, 0, st>>>(polls, error);
    TSP_CUDA(cudaGetLastError());
    return TSP_OK;
}

int launch_f16_to_f32(const void* in, uint64_t in_stride, float* out, uint64_t out_stride, uint32_t rows, uint32_t cols,
                      cudaStream_t st) {
    dim3 grid((cols + 1023) / 1024, rows);
    TSP_CUDA(launch_pdl(rows_f16_to_f32_kernel, grid, dim3(256), 0, st, static_cast<const __half*>(in), in_stride, out, out_stride, rows, cols));
    return TSP_OK;
}

int launch_dequant(uint32_t type, uint32_t layout, const uint8_t* expert, uint64_t total_blocks, float* out,
                   uint32_t* error, cudaStream_t st) {
    if (type == TSP_TYPE_Q4_K) dequant_q4k_kernel<<<static_cast<unsigned>(total_blocks), 256, 0, st>>>(expert, layout, total_blocks, out, error);
    else dequant_q8_kernel<<<static_cast<unsigned>((total_blocks + 7) / 8), 256, 0, st>>>(expert, layout, total_blocks, out, error);
    TSP_CUDA(cudaGetLastError());
    return TSP_OK;
}

}  // namespace tsp
