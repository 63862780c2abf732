// Expert-parallel MoE layer: slab pack / unpack kernels, the final mixture, and the step sequenced on one stream with two
// NCCL exchanges (all-to-all dispatch of token rows, per-peer send/recv of partial sums). Compute on the owners goes through
// the same C entry points as the one-GPU layer (libtsp_moe.so); this library adds only what the exchange needs.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <nccl.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "tsp_ep.h"

namespace {

thread_local char g_ep_message[512] = "";

int ep_fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_ep_message, sizeof g_ep_message, fmt, ap);
    va_end(ap);
    return code;
}
#define EP_REQUIRE(cond, ...) do { if (!(cond)) return ep_fail(TSP_E_ARG, __VA_ARGS__); } while (0)
#define EP_CUDA(expr) do { cudaError_t e_ = (expr); if (e_ != cudaSuccess) return ep_fail(TSP_E_CUDA, "CUDA error %d (%s) at %s", int(e_), cudaGetErrorString(e_), #expr); } while (0)
#define EP_NCCL(expr) do { ncclResult_t r_ = (expr); if (r_ != ncclSuccess) return ep_fail(TSP_E_CUDA, "NCCL error %d (%s) at %s", int(r_), ncclGetErrorString(r_), #expr); } while (0)
#define EP_TSP(expr) do { int rc_ = (expr); if (rc_ != TSP_OK) return ep_fail(rc_, "%s", tsp_last_error()); } while (0)

constexpr uint32_t kMetaOffset = 256;   // bytes of a slab before its routing rows: word 0 = row count

struct SlabGeometry {
    uint64_t row_bytes, slab_bytes;
    uint32_t header_rows, rows;   // rows = header_rows + tokens
};
SlabGeometry slab_geometry(uint32_t tokens, uint32_t channels, uint32_t selected) {
    SlabGeometry g;
    g.row_bytes = uint64_t(channels) * 2;
    const uint64_t meta = kMetaOffset + uint64_t(tokens) * selected * 8;
    g.header_rows = uint32_t((meta + g.row_bytes - 1) / g.row_bytes);
    g.rows = g.header_rows + tokens;
    g.slab_bytes = uint64_t(g.rows) * g.row_bytes;
    return g;
}

__device__ __forceinline__ uint32_t destination(uint32_t place, uint32_t rank) {
    const uint32_t owner = place >> 16;
    return owner == TSP_EP_REPLICATED ? rank : owner;
}

// One block per destination rank: pos[g][t] = position of token t among the tokens with a route to g (ascending token
// order: a stable compaction, no atomics), -1 for the others; the slab's count word.
__global__ void __launch_bounds__(1024)
ep_plan_kernel(const uint32_t* __restrict__ ids, const uint32_t* __restrict__ place, uint32_t tokens, uint32_t selected, uint32_t rank,
               int32_t* __restrict__ pos, uint8_t* __restrict__ slabs, uint64_t slab_bytes) {
    __shared__ uint32_t warp_sum[32];
    const uint32_t g = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t carry = 0;
    for (uint32_t base = 0; base < tokens; base += 1024) {
        const uint32_t t = base + tid;
        bool mine = false;
        if (t < tokens)
            for (uint32_t k = 0; k < selected; ++k) mine |= destination(place[ids[uint64_t(t) * selected + k]], rank) == g;
        const uint32_t ballot = __ballot_sync(0xffffffffu, mine);
        const uint32_t prefix = __popc(ballot & ((1u << lane) - 1u));
        if (lane == 0) warp_sum[warp] = __popc(ballot);
        __syncthreads();
        uint32_t before = 0, total = 0;
        for (uint32_t i = 0; i < 32; ++i) { if (i < warp) before += warp_sum[i]; total += warp_sum[i]; }
        if (t < tokens) pos[uint64_t(g) * tokens + t] = mine ? int32_t(carry + before + prefix) : -1;
        carry += total;
        __syncthreads();
    }
    if (tid == 0) *reinterpret_cast<uint32_t*>(slabs + g * slab_bytes) = carry;
}

// grid (tokens, world): the token's row and its routing row into the slab of every rank it has a route to
__global__ void __launch_bounds__(256)
ep_pack_kernel(const uint32_t* __restrict__ ids, const float* __restrict__ weights, const uint8_t* __restrict__ x16, uint64_t x_stride,
               const uint32_t* __restrict__ place, uint32_t tokens, uint32_t channels, uint32_t selected, uint32_t rank, int k_ordered,
               const int32_t* __restrict__ pos, uint8_t* __restrict__ slabs, uint64_t slab_bytes, uint32_t header_rows) {
    const uint32_t t = blockIdx.x, g = blockIdx.y;
    const int32_t j = pos[uint64_t(g) * tokens + t];
    if (j < 0) return;
    uint8_t* slab = slabs + g * slab_bytes;
    const uint4* src = reinterpret_cast<const uint4*>(x16 + t * x_stride);
    uint4* dst = reinterpret_cast<uint4*>(slab + (uint64_t(header_rows) + j) * channels * 2);
    for (uint32_t k8 = threadIdx.x; k8 < channels / 8; k8 += blockDim.x) {
        uint4 v = src[k8];
        if (k_ordered)   // the order inside each run of 8 that the tensor-core tiles use: 0,2,1,3,4,6,5,7
            v = make_uint4(__byte_perm(v.x, v.y, 0x5410), __byte_perm(v.x, v.y, 0x7632), __byte_perm(v.z, v.w, 0x5410), __byte_perm(v.z, v.w, 0x7632));
        dst[k8] = v;
    }
    if (threadIdx.x < selected) {
        const uint32_t k = threadIdx.x, pl = place[ids[uint64_t(t) * selected + k]];
        const bool mine = destination(pl, rank) == g;
        uint32_t* mid = reinterpret_cast<uint32_t*>(slab + kMetaOffset);
        float* mw = reinterpret_cast<float*>(slab + kMetaOffset + uint64_t(tokens) * selected * 4);
        mid[uint64_t(j) * selected + k] = mine ? (pl & 0xffffu) : 0xffffffffu;
        mw[uint64_t(j) * selected + k] = mine ? weights[uint64_t(t) * selected + k] : 0.f;
    }
}

// Dense routing tables over the row space of all received slabs: row r = p * rows_per_slab + i is token row i - header_rows of
// the slab from rank p when that is below the slab's count, otherwise it has no routes.
__global__ void __launch_bounds__(256)
ep_unpack_kernel(const uint8_t* __restrict__ slabs, uint64_t slab_bytes, uint32_t tokens, uint32_t selected, uint32_t header_rows,
                 uint32_t rows_per_slab, uint64_t total, uint32_t* __restrict__ ids_all, float* __restrict__ w_all) {
    const uint64_t at = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (at >= total) return;
    const uint32_t row = uint32_t(at / selected), k = uint32_t(at % selected);
    const uint32_t p = row / rows_per_slab, i = row % rows_per_slab;
    const uint8_t* slab = slabs + p * slab_bytes;
    const uint32_t count = *reinterpret_cast<const uint32_t*>(slab);
    uint32_t id = 0xffffffffu;
    float w = 0.f;
    if (i >= header_rows && i - header_rows < count && count <= tokens) {
        const uint32_t j = i - header_rows;
        id = reinterpret_cast<const uint32_t*>(slab + kMetaOffset)[uint64_t(j) * selected + k];
        w = reinterpret_cast<const float*>(slab + kMetaOffset + uint64_t(tokens) * selected * 4)[uint64_t(j) * selected + k];
    }
    ids_all[at] = id;
    w_all[at] = w;
}

// out[t][c] = sigmoid(w_sr . x[t]) * shared[t][c] + sum over ranks g (ascending) of the partial sum g returned for token t
// `own`: this rank's own partial rows (they never travel); the other ranks' rows are read from `ret`. Eight channels per thread
// step (16-byte loads of every rank's row), ranks added in ascending order.
template <bool P16>
__global__ void __launch_bounds__(256)
ep_finish_kernel(const uint8_t* __restrict__ ret, uint64_t ret_peer_bytes, const uint8_t* __restrict__ own, uint32_t rank, const int32_t* __restrict__ pos,
                 uint32_t world, uint32_t tokens, uint32_t channels, const float* __restrict__ shared, const float* __restrict__ shared_router,
                 const __half* __restrict__ x16, uint64_t x_stride, __half* __restrict__ out16, uint64_t out_stride, uint32_t* error) {
    __shared__ float partial[8];
    __shared__ float gate_s;
    __shared__ int32_t pos_s[64];
    const uint32_t t = blockIdx.x, tid = threadIdx.x;
    if (tid < world) pos_s[tid] = pos[uint64_t(tid) * tokens + t];
    float gate = 1.f;
    if (shared_router) {
        const __half* xr = reinterpret_cast<const __half*>(reinterpret_cast<const char*>(x16) + t * x_stride);
        float acc = 0.f;
        for (uint32_t c = tid; c < channels; c += 256) acc = fmaf(shared_router[c], __half2float(xr[c]), acc);
        for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if ((tid & 31) == 0) partial[tid >> 5] = acc;
        __syncthreads();
        if (tid == 0) {
            float s = 0.f;
            for (int i = 0; i < 8; ++i) s += partial[i];
            if ((__float_as_uint(s) & 0x7f800000u) == 0x7f800000u && error) atomicOr(error, TSP_ERR_NONFINITE);
            gate_s = s >= 0.f ? 1.f / (1.f + expf(-s)) : expf(s) / (1.f + expf(s));
        }
        __syncthreads();
        gate = gate_s;
    } else {
        __syncthreads();
    }
    bool bad = false;
    for (uint32_t c = tid * 8; c < channels; c += 256 * 8) {   // channels % 8 == 0 (checked by the entry point)
        const float4 s0 = *reinterpret_cast<const float4*>(shared + uint64_t(t) * channels + c), s1 = *reinterpret_cast<const float4*>(shared + uint64_t(t) * channels + c + 4);
        float v[8] = {gate * s0.x, gate * s0.y, gate * s0.z, gate * s0.w, gate * s1.x, gate * s1.y, gate * s1.z, gate * s1.w};
        for (uint32_t g = 0; g < world; ++g) {
            const int32_t j = pos_s[g];
            if (j < 0) continue;
            const uint8_t* row = (g == rank ? own : ret + g * ret_peer_bytes) + uint64_t(j) * channels * (P16 ? 2 : 4);
            if (P16) {
                const uint4 h = *reinterpret_cast<const uint4*>(row + c * 2ull);
                const uint32_t w4[4] = {h.x, h.y, h.z, h.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) { const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w4[q])); v[2 * q] += f.x; v[2 * q + 1] += f.y; }
            } else {
                const float4 a = *reinterpret_cast<const float4*>(row + c * 4ull), b4 = *reinterpret_cast<const float4*>(row + c * 4ull + 16);
                v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w; v[4] += b4.x; v[5] += b4.y; v[6] += b4.z; v[7] += b4.w;
            }
        }
        uint32_t h[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            bad |= (__float_as_uint(v[2 * q]) & 0x7f800000u) == 0x7f800000u || (__float_as_uint(v[2 * q + 1]) & 0x7f800000u) == 0x7f800000u;
            const __half2 t2 = __floats2half2_rn(v[2 * q], v[2 * q + 1]);
            h[q] = *reinterpret_cast<const uint32_t*>(&t2);
        }
        *reinterpret_cast<uint4*>(reinterpret_cast<char*>(out16) + t * out_stride + c * 2ull) = make_uint4(h[0], h[1], h[2], h[3]);
    }
    if (bad && error) atomicOr(error, TSP_ERR_NONFINITE);
}

struct Carve {
    uint8_t* base; uint64_t at = 0;
    template <typename T> T* take(uint64_t bytes) { T* p = reinterpret_cast<T*>(base + at); at += (bytes + 1023) & ~uint64_t(1023); return p; }
};

struct Plan {
    SlabGeometry sg;
    uint32_t rows_all;       // rows of the received row space: world * sg.rows
    uint64_t routes_all;     // rows_all * selected
    uint64_t total;
    // offsets into the scratch buffer
    uint32_t *ids, *ids_all, *token_map, *counts, *tasks, *offsets;
    int32_t* pos;
    float *weights, *w_all, *x32_all, *hidden, *routed, *partial, *x32_local, *shared_hidden, *shared_out;
    uint8_t *send, *recv, *ret, *xp, *hp, *routed16, *partial16, *xk_local, *s_hp;
};

Plan make_plan(uint8_t* base, uint32_t T, uint32_t C, uint32_t H, uint32_t Eloc, uint32_t K, uint32_t N, bool prefill) {
    Plan p{};
    p.sg = slab_geometry(T, C, K);
    p.rows_all = N * p.sg.rows;
    p.routes_all = uint64_t(p.rows_all) * K;
    Carve c{base};
    const uint64_t R = p.rows_all, RK = p.routes_all;
    p.ids = c.take<uint32_t>(uint64_t(T) * K * 4);
    p.weights = c.take<float>(uint64_t(T) * K * 4);
    p.pos = c.take<int32_t>(uint64_t(N) * T * 4);
    p.send = c.take<uint8_t>(N * p.sg.slab_bytes);
    p.recv = c.take<uint8_t>(N * p.sg.slab_bytes);
    p.ids_all = c.take<uint32_t>(RK * 4);
    p.w_all = c.take<float>(RK * 4);
    p.token_map = c.take<uint32_t>(uint64_t(Eloc) * R * 4);
    p.counts = c.take<uint32_t>(uint64_t(Eloc) * 4);
    const uint32_t tile = prefill ? TSP_GROUPED_TILE : TSP_GEMV_TILE;
    p.tasks = c.take<uint32_t>(tsp_moe_tasks_words(uint32_t(R), Eloc, K, tile) * 4);
    p.offsets = c.take<uint32_t>((uint64_t(Eloc) + 5) * 4);
    p.shared_out = c.take<float>(uint64_t(T) * C * 4);
    p.ret = c.take<uint8_t>(uint64_t(N) * T * C * (prefill ? 2 : 4));
    if (prefill) {
        p.xp = c.take<uint8_t>(RK * C * 2);
        p.hp = c.take<uint8_t>(RK * H * 2);
        p.routed16 = c.take<uint8_t>(RK * C * 2);
        p.partial16 = c.take<uint8_t>(R * C * 2);
        p.xk_local = c.take<uint8_t>(uint64_t(T) * C * 2);
        p.s_hp = c.take<uint8_t>(uint64_t(T) * H * 2);
    } else {
        p.x32_all = c.take<float>(R * C * 4);
        p.hidden = c.take<float>(RK * H * 4);
        p.routed = c.take<float>(RK * C * 4);
        p.partial = c.take<float>(R * C * 4);
        p.x32_local = c.take<float>(uint64_t(T) * C * 4);
        p.shared_hidden = c.take<float>(uint64_t(T) * H * 4);
    }
    p.total = c.at;
    return p;
}

}  // namespace

struct tsp_ep_ctx {
    ncclComm_t comm;
    int rank, world, device;
};

extern "C" {

int tsp_ep_unique_id(uint8_t* id) {
    EP_REQUIRE(id, "unique id: null buffer");
    static_assert(sizeof(ncclUniqueId) <= TSP_EP_ID_BYTES, "id buffer too small");
    ncclUniqueId u;
    EP_NCCL(ncclGetUniqueId(&u));
    memset(id, 0, TSP_EP_ID_BYTES);
    memcpy(id, &u, sizeof u);
    return TSP_OK;
}

int tsp_ep_create(const uint8_t* id, int rank, int world, tsp_ep_ctx** out) {
    EP_REQUIRE(id && out && world >= 1 && world <= 64 && rank >= 0 && rank < world, "context: bad rank / world");
    ncclUniqueId u;
    memcpy(&u, id, sizeof u);
    tsp_ep_ctx* ctx = new tsp_ep_ctx{};
    ctx->rank = rank; ctx->world = world;
    if (cudaGetDevice(&ctx->device) != cudaSuccess) { delete ctx; return ep_fail(TSP_E_CUDA, "no usable CUDA device"); }
    const ncclResult_t r = ncclCommInitRank(&ctx->comm, world, u, rank);
    if (r != ncclSuccess) { delete ctx; return ep_fail(TSP_E_CUDA, "ncclCommInitRank failed: %s", ncclGetErrorString(r)); }
    *out = ctx;
    return TSP_OK;
}

int tsp_ep_destroy(tsp_ep_ctx* ctx) {
    if (!ctx) return TSP_OK;
    ncclCommDestroy(ctx->comm);
    delete ctx;
    return TSP_OK;
}

uint32_t tsp_ep_slab_header_rows(uint32_t tokens, uint32_t channels, uint32_t selected) {
    if (!tokens || !channels || !selected) return 0;
    return slab_geometry(tokens, channels, selected).header_rows;
}

uint64_t tsp_ep_slab_bytes(uint32_t tokens, uint32_t channels, uint32_t selected) {
    if (!tokens || !channels || !selected) return 0;
    return slab_geometry(tokens, channels, selected).slab_bytes;
}

uint64_t tsp_ep_scratch_bytes(uint32_t tokens, uint32_t channels, uint32_t hidden, uint32_t experts, uint32_t local_experts, uint32_t selected,
                              uint32_t world, int prefill) {
    if (!tokens || !channels || !hidden || !experts || !local_experts || !selected || !world) return 0;
    return make_plan(nullptr, tokens, channels, hidden, local_experts, selected, world, prefill != 0).total;
}

int tsp_ep_pack(const uint32_t* d_ids, const float* d_weights, const void* d_x16, uint64_t x_stride, const uint32_t* d_place, uint32_t tokens,
                uint32_t channels, uint32_t selected, uint32_t rank, uint32_t world, int k_ordered, int32_t* d_pos, void* d_slabs, void* stream) {
    EP_REQUIRE(d_ids && d_weights && d_x16 && d_place && d_pos && d_slabs, "pack: null buffer");
    EP_REQUIRE(tokens >= 1 && tokens <= 65535 && channels >= 8 && channels % 8 == 0 && selected >= 1 && selected <= 64 && world >= 1 && world <= 64 &&
               rank < world, "pack: invalid shape");
    EP_REQUIRE(x_stride >= channels * 2ull && x_stride % 16 == 0 && reinterpret_cast<uintptr_t>(d_x16) % 16 == 0, "pack: rows must be 16-byte aligned");
    const SlabGeometry sg = slab_geometry(tokens, channels, selected);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ep_plan_kernel<<<world, 1024, 0, st>>>(d_ids, d_place, tokens, selected, rank, d_pos, static_cast<uint8_t*>(d_slabs), sg.slab_bytes);
    EP_CUDA(cudaGetLastError());
    ep_pack_kernel<<<dim3(tokens, world), 256, 0, st>>>(d_ids, d_weights, static_cast<const uint8_t*>(d_x16), x_stride, d_place, tokens, channels, selected,
                                                         rank, k_ordered, d_pos, static_cast<uint8_t*>(d_slabs), sg.slab_bytes, sg.header_rows);
    EP_CUDA(cudaGetLastError());
    return TSP_OK;
}

int tsp_ep_unpack(const void* d_slabs, uint32_t tokens, uint32_t channels, uint32_t selected, uint32_t world, uint32_t* d_ids_all,
                  float* d_weights_all, void* stream) {
    EP_REQUIRE(d_slabs && d_ids_all && d_weights_all && tokens >= 1 && channels >= 8 && selected >= 1 && selected <= 64 && world >= 1 && world <= 64,
               "unpack: null buffer or invalid shape");
    const SlabGeometry sg = slab_geometry(tokens, channels, selected);
    const uint64_t total = uint64_t(world) * sg.rows * selected;
    ep_unpack_kernel<<<unsigned((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint8_t*>(d_slabs), sg.slab_bytes, tokens,
                                                                                                 selected, sg.header_rows, sg.rows, total, d_ids_all, d_weights_all);
    EP_CUDA(cudaGetLastError());
    return TSP_OK;
}

int tsp_ep_moe_layer(tsp_ep_ctx* ctx, const tsp_ep_layer* L, void* d_scratch, uint64_t scratch_bytes, const void* d_x16, uint64_t x_stride,
                     const float* d_logits, uint64_t logits_stride, uint32_t tokens, uint32_t channels, uint32_t hidden, uint32_t experts,
                     uint32_t selected, uint32_t mode, int normalize, int prefill, void* d_out16, uint64_t out_stride, uint32_t* d_error, void* stream) {
    EP_REQUIRE(ctx && L && d_scratch && d_x16 && d_logits && d_out16 && L->d_place, "layer: null argument");
    EP_REQUIRE(tokens >= 1 && channels % 8 == 0 && L->local_experts >= 1, "layer: invalid shape");
    EP_REQUIRE((reinterpret_cast<uintptr_t>(d_out16) | out_stride) % 16 == 0, "layer: output rows must be 16-byte aligned");
    EP_REQUIRE(reinterpret_cast<uintptr_t>(d_scratch) % 1024 == 0, "layer: the scratch buffer must be 1024-byte aligned");
    const uint32_t N = uint32_t(ctx->world), rank = uint32_t(ctx->rank), T = tokens, C = channels, H = hidden, K = selected, El = L->local_experts;
    const bool pf = prefill != 0;
    const Plan p = make_plan(static_cast<uint8_t*>(d_scratch), T, C, H, El, K, N, pf);
    EP_REQUIRE(p.total <= scratch_bytes, "layer: scratch of %llu bytes, %llu needed", (unsigned long long)scratch_bytes, (unsigned long long)p.total);
    EP_REQUIRE(p.rows_all <= 65535 || pf, "layer: too many rows for the decode-size path");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const tsp_moe_weights& w = L->local;
    const uint64_t rb = p.sg.row_bytes;

    // ---- source side: route, pack, dispatch
    EP_TSP(tsp_moe_route(d_logits, logits_stride, T, experts, K, mode, normalize, p.ids, p.weights, d_error, st));
    if (int rc = tsp_ep_pack(p.ids, p.weights, d_x16, x_stride, L->d_place, T, C, K, rank, N, pf ? 1 : 0, p.pos, p.send, st)) return rc;
    EP_NCCL(ncclAlltoAll(p.send, p.recv, p.sg.slab_bytes, ncclUint8, ctx->comm, st));

    // ---- owner side: the received rows form one row space of N * (header rows + T) rows of `rb` bytes
    const uint32_t R = p.rows_all;
    if (int rc = tsp_ep_unpack(p.recv, T, C, K, N, p.ids_all, p.w_all, st)) return rc;
    const uint32_t tile = pf ? TSP_GROUPED_TILE : TSP_GEMV_TILE;
    EP_TSP(tsp_moe_permute_local(p.ids_all, R, 0, El, K, tile, p.token_map, p.counts, p.tasks, d_error, st));
    if (pf) {
        EP_TSP(tsp_moe_route_offsets(p.counts, El, p.offsets, st));
        EP_TSP(tsp_moe_gather_rows16(p.recv, rb, p.token_map, p.offsets, El, R, K, C, p.xp, rb, st));
        EP_TSP(tsp_moe_rows_f16k(d_x16, x_stride, 1, T, C, p.xk_local, rb, d_error, st));
        EP_TSP(tsp_moe_grouped_gate_up(&w.gate, &w.up, &w.shared_gate, &w.shared_up, p.xp, rb, p.xk_local, rb, T, R, K, p.token_map, p.counts, p.tasks,
                                       p.offsets, p.hp, H * 2ull, p.s_hp, H * 2ull, d_error, st));
        EP_TSP(tsp_moe_grouped_down(&w.down, &w.shared_down, p.hp, H * 2ull, R, K, p.token_map, p.counts, p.tasks, p.offsets, p.routed16, rb, 1, p.s_hp,
                                    H * 2ull, T, p.shared_out, C * 4ull, d_error, st));
        // per received row: the weighted sum of its local routes, as binary16 (zero weights mark routes served elsewhere)
        EP_TSP(tsp_moe_combine(p.routed16, rb, 1, p.w_all, nullptr, 0, nullptr, nullptr, 0, 0, nullptr, R, C, K, nullptr, 0, p.partial16, rb, d_error, st));
    } else {
        // the routed experts work on the received rows, the shared expert on this rank's own rows: both in the same two launches
        EP_TSP(tsp_rows_f16_to_f32(p.recv, rb, p.x32_all, C * 4ull, R, C, st));
        EP_TSP(tsp_rows_f16_to_f32(d_x16, x_stride, p.x32_local, C * 4ull, T, C, st));
        EP_TSP(tsp_moe_gate_up_swiglu_shared_rows(&w.gate, &w.up, &w.shared_gate, &w.shared_up, p.x32_all, C * 4ull, nullptr, 0, R, K, p.token_map, p.counts,
                                                  p.tasks, p.hidden, H * 4ull, p.x32_local, C * 4ull, T, p.shared_hidden, H * 4ull, 1, d_error, st));
        EP_TSP(tsp_moe_project_shared_rows(&w.down, &w.shared_down, p.hidden, H * 4ull, p.shared_hidden, H * 4ull, T, R, K, p.token_map, p.counts, p.tasks,
                                           p.routed, C * 4ull, p.shared_out, C * 4ull, d_error, st));
        EP_TSP(tsp_moe_combine(p.routed, C * 4ull, 0, p.w_all, nullptr, 0, nullptr, nullptr, 0, 0, nullptr, R, C, K, p.partial, C * 4ull, nullptr, 0, d_error, st));
    }

    // ---- combine: the partial sums of slab q's rows go back to rank q
    const uint64_t es = pf ? 2 : 4, peer_bytes = uint64_t(T) * C * es;
    const uint8_t* partial = pf ? p.partial16 : reinterpret_cast<const uint8_t*>(p.partial);
    EP_NCCL(ncclGroupStart());
    for (uint32_t q = 0; q < N; ++q) {
        const uint8_t* src = partial + (uint64_t(q) * p.sg.rows + p.sg.header_rows) * C * es;
        if (q == rank) continue;
        EP_NCCL(ncclSend(src, peer_bytes, ncclUint8, int(q), ctx->comm, st));
        EP_NCCL(ncclRecv(p.ret + q * peer_bytes, peer_bytes, ncclUint8, int(q), ctx->comm, st));
    }
    EP_NCCL(ncclGroupEnd());
    // ---- source side: gated shared expert + partial sums in ascending rank order (this rank's own rows straight from `partial`)
    const uint8_t* own = partial + (uint64_t(rank) * p.sg.rows + p.sg.header_rows) * C * es;
    if (pf) ep_finish_kernel<true><<<T, 256, 0, st>>>(p.ret, peer_bytes, own, rank, p.pos, N, T, C, p.shared_out, w.d_shared_router, static_cast<const __half*>(d_x16),
                                                      x_stride, static_cast<__half*>(d_out16), out_stride, d_error);
    else ep_finish_kernel<false><<<T, 256, 0, st>>>(p.ret, peer_bytes, own, rank, p.pos, N, T, C, p.shared_out, w.d_shared_router, static_cast<const __half*>(d_x16),
                                                    x_stride, static_cast<__half*>(d_out16), out_stride, d_error);
    EP_CUDA(cudaGetLastError());
    return TSP_OK;
}

const char* tsp_ep_last_error(void) { return g_ep_message; }

}  // extern "C"
