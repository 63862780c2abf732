// Prefill-size grouped expert GEMMs on the 5th-generation tensor cores (tcgen05) for sm_100a.
//
// One launch computes, for every task of <= 256 routes of one expert (two sub-tiles of <= 128 token columns), either
//   gate-up:  H[pos][h]   = silu(W_gate[h] . x[token]) * (W_up[h] . x[token])
//   down:     Y[route][c] = W_down[c] . H[pos]
// with the weights as the M operand (128 weight rows per item fill the MMA's M extent whatever the number of tokens), the
// tokens as the N operand (32, 64 or 128 columns per sub-tile) and K walked in chunks of 64.
//
//   * A dequantised weight chunk is used for BOTH sub-tiles of a task before it is released: an expert with many routes
//     pays the dequantisation once per 256 routes. Each sub-tile has its own accumulator (128 columns of tensor memory);
//     two such pairs are double-buffered (512 columns), so the epilogue of an item runs under the MMAs of the next.
//   * One pipeline stage = one K chunk = {dequantised weight chunk, activation tile of sub-tile 0, of sub-tile 1}, filled by
//     the dequant warps and the activation producer, emptied by ONE commit. The thread that issues the MMAs does one wait,
//     four MMAs (N = 256 when both sub-tiles are full: their tiles are adjacent) and one commit per chunk: with separate rings
//     for weights and activations its waits and commits, not the tensor pipe, set the pace (measured: removing the MMAs
//     altogether made the launch only 30 % shorter).
//   * Gate-up items hold 64 hidden units as 128 A rows: inside every group of 32 rows (one tensor-memory lane quarter)
//     rows 0..15 are gate rows and rows 16..31 the up rows of the same 16 units, so SwiGLU is a lane exchange inside one
//     warp and one accumulator serves both matrices (a 16 KB A stage per chunk, four stages).
//   * Activation tiles are plain tile copies (one `cp.async.bulk.tensor` per tile and K chunk) of rows kept in permuted
//     position order: the routed copy of the input rows for gate-up (written once per layer by `gather_rows16_kernel`; the
//     shared expert's tasks read the input rows themselves), the hidden rows for down. Fetching rows by token id inside the
//     GEMM (`tile::gather4`, four rows per instruction) was measured and dropped: one such instruction costs the issuing
//     warp about 200 cycles, so a 128-column tile needs 6400 cycles of issue per K chunk against 256 cycles of MMA.
//   * Items (task x block of weight rows) are handed out at run time: one thread takes the next index from a global counter
//     and publishes it to the CTA's roles through a small ring, so CTAs whose items are heavy (256 routes) simply take fewer.
//
// Roles inside a CTA (one persistent CTA per SM):
//   warp 0      TMA producer of the quantised planes: Pack v3 planar code lines + 6-bit factor bytes of one super-block
//               (256 columns of K) per quant stage; the (d, dmin) pairs once per item.
//   warp 1      allocates tensor memory, issues tcgen05.mma (one elected lane), commits to mbarriers.
//   warps 2..9  dequantise: a thread owns one weight row and every other K chunk (threads 0..127 the even chunks, 128..255
//               the odd ones): 32 code bytes -> 64 binary16 weights written as one 128-byte row of the K-major,
//               128-byte-swizzled operand tile. Per group of 32 weights the value staged is
//               RN16((q - 8) * RN16(d*sc) + RN16(8*d*sc - dmin*mn)): the centred code keeps the products small, so the three
//               roundings cost about 1.5x the error of rounding the exact value once (measured by the tile hook below).
//   warp 10     activation producer.
//   warps 11..18 epilogue (two per tensor-memory lane quarter): tcgen05.ld of their 32 accumulator lanes, SwiGLU / store.
// Accumulation is FP32 in tensor memory. Operands are binary16 (kind::f16, f16 inputs): the activations of this path are
// binary16-exact, and Q4_K values keep 11 significant bits instead of bf16's 8.
// Every mbarrier wait is bounded; a timeout sets TSP_ERR_TIMEOUT, and every path still frees the tensor memory.
#include <cuda.h>

#include "tsp_common.cuh"

namespace tsp {

int get_tensor_map_bytes(const void* base, uint32_t rank, const uint64_t* dims, const uint64_t* strides, const uint32_t* box,
                         bool swizzle128, CUtensorMap* out);

// ---------------------------------------------------------------------------------------------
// tcgen05 / TMEM wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc], kind::f16, one CTA
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrive on an mbarrier when all MMAs issued so far by this thread have completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 lanes x 32 consecutive columns -> 32 registers per thread
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_4d_g(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void tma_load_5d_g(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
                 ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
                 : "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile whose rows are 128 bytes (64 binary16) in the 128-byte swizzle:
// start address >> 4, leading byte offset (unused for this layout) 1, stride byte offset 1024 (eight rows), descriptor
// version 1 (sm_100), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc_k128(const void* smem_tile) {
    const uint64_t addr = smem_u32(smem_tile);
    return ((addr & 0x3FFFFull) >> 4) | (1ull << 16) | (uint64_t(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor for kind::f16: D = FP32, A = B = binary16, both K-major, M x N tile.
__host__ __device__ constexpr uint32_t umma_idesc_f16(uint32_t m, uint32_t n) {
    return (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (0u << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

constexpr uint32_t kDqWarps = 8;           // dequantise warps: 256 threads = 128 weight rows x {even, odd} K chunks
constexpr uint32_t kEpWarps = 8;           // epilogue warps: two per tensor-memory lane quarter, taking the 32-column batches in turn
constexpr uint32_t kGWarps = 3 + kDqWarps + kEpWarps;   // weight producer, MMA, dequant warps, activation producer, epilogue warps
constexpr uint32_t kTaskRoutes = TSP_GROUPED_TILE;      // routes per task (two sub-tiles)
constexpr uint32_t kSub = 128;             // token columns per sub-tile (N extent at most)
constexpr uint32_t kRowsM = 128;           // A rows per item (M)
constexpr uint32_t kStages = 3;            // K chunks in flight: a stage holds the dequantised weight chunk AND the activation tiles it meets
constexpr uint32_t kStageBytes = 3 * 16384;   // [A: 128 rows x 128 B][B sub-tile 0][B sub-tile 1]
constexpr uint32_t kEpTileBytes = 32 * 144;   // per epilogue warp: 32 token rows of 32 FP32 values, rows padded by 16 bytes
static_assert(kTaskRoutes == 2 * kSub, "a task is two sub-tiles");

// Tensor maps of one launch: codes / factor bytes / (d, dmin) pairs with index 0 matrix A low ids, 1 A high ids, 2 B low ids,
// 3 B high ids, 4 shared-expert A, 5 shared-expert B. Activations: x[0..2] = tiles of 32 / 64 / 128 rows of the routed rows in
// permuted position order, x[3..5] the same over the shared expert's rows (row = token).
struct alignas(64) GroupedMaps { CUtensorMap q[6], f[6], d[6], x[6]; };

struct GroupedParams {
    uint32_t split, experts;
    uint32_t nblk;                 // quant-stage loads per item: super-blocks per weight row (K / 256); Q8_0: spans of four blocks (K / 128)
    uint32_t chunks;               // K chunks of 64 per item
    uint32_t row_blocks;           // items per task: hidden / 64 (gate-up) or rows / 128 (down)
    uint32_t merged, sh_merged;    // both matrices of an expert arrive with one copy per plane (routed experts; shared expert)
    // optional dense shared expert processed by the same launch after the routed tasks: every one of sh_tokens rows, in
    // row order (position = token = route id)
    uint32_t sh_tasks, sh_tokens;
    void* sh_out; uint64_t sh_out_stride_bytes;
    // routes
    uint32_t tokens, selected;     // rows of token_map per expert; routes per token row (route id = row * selected + slot)
    const uint32_t* tasks;         // {tasks, routes, (expert, start)...} with tasks of kTaskRoutes routes
    const uint32_t* counts;
    const uint32_t* offsets;       // first permuted position of each expert (hidden rows are kept in this order)
    const uint32_t* token_map;     // [expert][tokens] route ids in ascending order
    // output
    void* out; uint64_t out_stride_bytes;
    uint32_t out_f16;              // down: binary16 instead of FP32 route rows
    uint32_t* error;
    uint32_t* work_counter;        // next item index; zero when the launch starts (tsp_moe_route_offsets clears it)
    // shared-memory plan
    uint32_t off_q, q_stage_bytes, off_d, d_stage_bytes, dm_mat_bytes, off_st, off_ep;
};

// bounded wait with a short limit: a stalled pipeline ends in tens of milliseconds, never hangs
__device__ __forceinline__ bool gwait(uint64_t* bar, uint32_t parity) { return mbar_wait(bar, parity, 1u << 21); }

struct GTask { uint32_t expert, start, count, row0; };

// A task of the shared expert carries the expert id p.experts (one past the routed ids).
__device__ __forceinline__ GTask gtask(const GroupedParams& p, uint32_t task) {
    GTask t;
    const uint32_t routed = p.tasks ? p.tasks[0] : 0u;
    if (task >= routed) {
        t.expert = p.experts;
        t.start = (task - routed) * kTaskRoutes;
        t.count = t.start < p.sh_tokens ? min(p.sh_tokens - t.start, kTaskRoutes) : 0u;
        t.row0 = t.start;
        return t;
    }
    t.expert = p.tasks[2 + 2 * task];
    t.start = p.tasks[3 + 2 * task];
    if (t.expert >= p.experts) { t.expert = 0; t.start = 0; t.count = 0; t.row0 = 0; return t; }
    const uint32_t c = p.counts[t.expert];
    t.count = c > t.start ? min(c - t.start, kTaskRoutes) : 0u;
    t.row0 = p.offsets[t.expert] + t.start;
    return t;
}
__device__ __forceinline__ uint32_t sub_count(const GTask& t, uint32_t g) { return g == 0 ? min(t.count, kSub) : (t.count > kSub ? t.count - kSub : 0u); }
__device__ __forceinline__ uint32_t sub_cols(uint32_t count) { return count <= 32 ? 32u : (count <= 64 ? 64u : 128u); }
__device__ __forceinline__ uint32_t sub_tiles(const GTask& t) { return t.count > kSub ? 2u : 1u; }

// ---------------------------------------------------------------------------------------------
// dequantisation of one 64-wide K chunk of one weight row (shared by the GEMM kernel and the tile hook)
// ---------------------------------------------------------------------------------------------
struct ChunkScale { __half2 s_lo, c_lo, s_hi, c_hi; };

// d, dmin: the super-block's binary16 pair as floats; scw / mnw: four scale / min bytes of which bytes `b`, `b + 1` belong to
// this chunk's two groups (low nibbles: group 2c, high nibbles: group 2c + 1). d*sc and dmin*mn are exact in FP32.
__device__ __forceinline__ ChunkScale chunk_scale(float d, float dmin, uint32_t scw, uint32_t mnw, uint32_t b) {
    // byte -> float through the 2^23 magic number (0x4B0000bb = 2^23 + bb), folded into one FMA each
    const uint32_t sel_lo = 0x7440u + b, sel_hi = sel_lo + 1u;
    const float dn = d * -8388608.f, mn = dmin * -8388608.f;
    const float s_lo = fmaf(d, __uint_as_float(__byte_perm(scw, 0x4b000000u, sel_lo)), dn);
    const float s_hi = fmaf(d, __uint_as_float(__byte_perm(scw, 0x4b000000u, sel_hi)), dn);
    const float m_lo = fmaf(dmin, __uint_as_float(__byte_perm(mnw, 0x4b000000u, sel_lo)), mn);
    const float m_hi = fmaf(dmin, __uint_as_float(__byte_perm(mnw, 0x4b000000u, sel_hi)), mn);
    ChunkScale cs;
    cs.s_lo = __float2half2_rn(s_lo); cs.c_lo = __float2half2_rn(fmaf(8.f, s_lo, -m_lo));
    cs.s_hi = __float2half2_rn(s_hi); cs.c_hi = __float2half2_rn(fmaf(8.f, s_hi, -m_hi));
    return cs;
}

// Eight code bytes (words a, b = bytes 8qq..8qq+7 of the chunk's 32) -> the 8 weights of their low nibbles (`lo`: K positions
// 8qq..8qq+7 of the chunk) and the 8 of their high nibbles (`hi`: K positions 32+8qq..). Inside each run of 8 the values sit
// in the order 0,2,1,3,4,6,5,7, the order every K-major operand of these kernels uses: a 32-bit word of codes splits into
// binary16 pairs without byte shuffles.
__device__ __forceinline__ void dequant8(uint32_t a, uint32_t b, const ChunkScale& cs, uint4& lo, uint4& hi) {
    const __half2 k1032 = __float2half2_rn(1032.f), k72 = __float2half2_rn(72.f);
    const uint32_t src[4] = {a, a >> 8, b, b >> 8};
    uint32_t l[4], h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t lw = (src[i] & 0x000f000fu) | 0x64006400u;     // 1024 + q
        const uint32_t hw = (src[i] & 0x00f000f0u) | 0x54005400u;     //   64 + q
        const __half2 ql = __hsub2(*reinterpret_cast<const __half2*>(&lw), k1032);   // q - 8, exact
        const __half2 qh = __hsub2(*reinterpret_cast<const __half2*>(&hw), k72);
        const __half2 wl = __hfma2(ql, cs.s_lo, cs.c_lo), wh = __hfma2(qh, cs.s_hi, cs.c_hi);
        l[i] = *reinterpret_cast<const uint32_t*>(&wl);
        h[i] = *reinterpret_cast<const uint32_t*>(&wh);
    }
    lo = make_uint4(l[0], l[1], l[2], l[3]);
    hi = make_uint4(h[0], h[1], h[2], h[3]);
}

// Item hand-out. One thread (the weight producer) takes the next item index from the global counter, looks its task up and
// publishes both in a ring of kSched slots; the other 18 warps read it (one arrival per warp frees the slot). An index
// >= n_items ends every role.
constexpr uint32_t kSched = 4;
constexpr uint32_t kSchedReaders = 2 + kDqWarps + kEpWarps;   // MMA issuer, activation producer, dequant warps, epilogue warps
struct SchedItem { uint32_t item; GTask t; };
struct SchedReader {
    uint64_t* full; uint64_t* empty; const volatile uint32_t* slots;   // 8 words per slot: item, expert, start, count, row0
    uint32_t s = 0, ph = 0;
    // every lane of the warp calls this; item 0xffffffff when a bounded wait expired
    __device__ __forceinline__ SchedItem next(uint32_t lane) {
        const bool ok = mbar_wait(&full[s], ph, 1u << 21);
        SchedItem it;
        const volatile uint32_t* w = slots + s * 8;
        it.item = ok ? w[0] : 0xffffffffu;
        it.t.expert = w[1]; it.t.start = w[2]; it.t.count = w[3]; it.t.row0 = w[4];
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(&empty[s]);
        if (++s == kSched) { s = 0; ph ^= 1u; }
        return it;
    }
};

// GATEUP: two weight matrices (gate, up) interleaved 16 + 16 rows per lane quarter and the SwiGLU epilogue writing binary16
// hidden rows in permuted position order; otherwise one matrix and route rows scattered to their route ids.
// ENC selects the weight bytes:
//   kEncPlanar  Q4_K Pack v3 planes (codes, 16-byte factor records, (d, dmin) pairs);
//   kEncGguf    Q4_K plain 144-byte super-blocks (16-byte header: d, dmin, twelve bytes of packed 6-bit factors; then the 128
//               code bytes). The code map steps 144 bytes per super-block from the first block's byte 16, the factor map brings
//               the whole header, the (d, dmin) ring is left idle and the dequant warps unpack the factors (numeric.cpp:17-31);
//   kEncQ8      Q8_0 plain 34-byte blocks (binary16 scale, 32 signed codes; numeric.cpp:33-45). A quant stage holds four blocks
//               (136 bytes = two K chunks) of every row in a 144-byte line: 136 * span is 16-byte aligned for even spans only,
//               so odd spans are fetched from 8 bytes earlier and read from byte 8 of the line.
constexpr int kEncPlanar = 0, kEncGguf = 1, kEncQ8 = 2;

// One Q8_0 chunk (two blocks = 68 bytes starting at word WS of the 20 words `L`) -> the chunk's 128-byte A row. Block 0 starts on
// a word boundary (scale in the low half-word, codes two bytes off: realigned with funnel shifts), block 1 two bytes past one
// (scale in the high half-word, codes word-aligned). A code byte b becomes binary16 through 0x6400 | (b ^ 0x80) = 1152 + q, the
// subtraction is exact and d * q is rounded once: the staged value is RN16 of the exact weight.
template <uint32_t WS>
__device__ __forceinline__ bool q8_chunk_row(const uint32_t (&L)[20], uint8_t* arow, uint32_t sw) {
    const __half2 k1152 = __float2half2_rn(1152.f);
    const uint32_t s0 = L[WS] & 0xffffu, s1 = L[WS + 8] >> 16;
    const bool finite = (s0 & 0x7c00u) != 0x7c00u && (s1 & 0x7c00u) != 0x7c00u;
    const uint32_t dw0 = s0 | (s0 << 16), dw1 = s1 | (s1 << 16);
    const __half2 d0 = *reinterpret_cast<const __half2*>(&dw0), d1 = *reinterpret_cast<const __half2*>(&dw1);
#pragma unroll
    for (uint32_t u = 0; u < 8; ++u) {          // unit u: K positions 8u .. 8u+7 of the chunk
        uint32_t a, b;
        if (u < 4) { a = __funnelshift_r(L[WS + 2 * u], L[WS + 2 * u + 1], 16); b = __funnelshift_r(L[WS + 2 * u + 1], L[WS + 2 * u + 2], 16); }
        else { a = L[WS + 9 + 2 * (u - 4)]; b = L[WS + 10 + 2 * (u - 4)]; }
        a ^= 0x80808080u; b ^= 0x80808080u;
        const __half2 d = u < 4 ? d0 : d1;
        uint32_t w[4] = {__byte_perm(a, 0x64646464u, 0x4240), __byte_perm(a, 0x64646464u, 0x4341),
                         __byte_perm(b, 0x64646464u, 0x4240), __byte_perm(b, 0x64646464u, 0x4341)};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 v = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&w[i]), k1152), d);
            w[i] = *reinterpret_cast<const uint32_t*>(&v);
        }
        *reinterpret_cast<uint4*>(arow + ((u ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    return finite;
}

template <bool GATEUP, int ENC>
__global__ void __launch_bounds__(kGWarps * 32, 1) grouped_mma_kernel(const __grid_constant__ GroupedMaps maps, const GroupedParams p) {
    pdl_launch_dependents();
    extern __shared__ uint8_t gsm_raw[];
    uint8_t* gsm = gsm_raw + ((1024u - (smem_u32(gsm_raw) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(gsm);
    // rings: quantised super-blocks (2 stages, TMA), the (d, dmin) pairs of an item (2 stages, TMA), the K-chunk stages
    // (weight chunk from the dequant warps + activation tiles by TMA) and the item hand-out
    uint64_t *qfull = bars, *qempty = bars + 2, *dfull = bars + 4, *dempty = bars + 6, *full = bars + 8, *empty = full + kStages,
             *acc_full = empty + kStages, *acc_empty = acc_full + 2, *sfull = acc_empty + 2, *sempty = sfull + kSched;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gsm + 512);
    volatile uint32_t* sched_slots = reinterpret_cast<volatile uint32_t*>(gsm + 640);   // kSched x 8 words
    constexpr uint32_t NMAT = GATEUP ? 2 : 1;
    constexpr uint32_t RM = GATEUP ? 64 : 128;    // rows of ONE matrix in an item
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(&qfull[s], 1); mbar_init(&qempty[s], kDqWarps);
            mbar_init(&dfull[s], 1); mbar_init(&dempty[s], kDqWarps);
            mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], kEpWarps);
        }
        // a stage is full when the four dequant warps that own its chunk have written it and the activation bytes have landed
        for (uint32_t s = 0; s < kStages; ++s) { mbar_init(&full[s], kDqWarps / 2 + 1); mbar_init(&empty[s], 1); }
        for (uint32_t s = 0; s < kSched; ++s) { mbar_init(&sfull[s], 1); mbar_init(&sempty[s], kSchedReaders); }
        mbar_fence_init();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }   // two sets of two 128-column accumulators
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();   // everything above touched shared and tensor memory only

    constexpr bool GGUF = ENC == kEncGguf, Q8 = ENC == kEncQ8;
    const uint32_t routed_tasks = p.tasks ? p.tasks[0] : 0u;   // no table: a dense launch (the shared expert's tasks only)
    const uint32_t n_tasks = routed_tasks + p.sh_tasks;
    const uint32_t n_items = n_tasks * p.row_blocks;
    const uint32_t chunks_per_item = p.chunks;     // K chunks of 64 (an even number: a dequant thread's chunk parity is the same in every item)
    SchedReader sched{sfull, sempty, sched_slots};
    uint8_t* const stages = gsm + p.off_st;

    if (warp == 0) {
        // =========================== item hand-out + TMA producer of the quantised planes ===========================
        if (lane == 0) {
            bool ok = true;
            uint32_t qs = 0, qph = 0, ds = 0, dph = 0, cur = 0xffffffffu, ss = 0, sph = 0;
            GTask t{};
            while (ok) {
                ok = gwait(&sempty[ss], sph ^ 1u);
                if (!ok) break;
                uint32_t item = atomicAdd(p.work_counter, 1u);
                if (item >= n_items) item = 0xfffffffeu;            // the end marker (0xffffffff is reserved for an expired wait)
                else if (item / p.row_blocks != cur) { cur = item / p.row_blocks; t = gtask(p, cur); }
                volatile uint32_t* w = sched_slots + ss * 8;
                w[0] = item; w[1] = t.expert; w[2] = t.start; w[3] = t.count; w[4] = t.row0;
                mbar_arrive(&sfull[ss]);
                if (++ss == kSched) { ss = 0; sph ^= 1u; }
                if (item >= n_items) break;
                const uint32_t rb = item % p.row_blocks;
                const int r0 = static_cast<int>(rb * RM);
                const bool shared = t.expert >= p.experts;
                const bool hi = !shared && t.expert >= p.split;
                const int el = shared ? 0 : static_cast<int>(hi ? t.expert - p.split : t.expert);
                const uint32_t mi = shared ? 4u : (hi ? 1u : 0u);                 // map of matrix A; matrix B's is `ms` further
                const uint32_t ms = shared ? 1u : 2u;
                const uint32_t ncopy = (NMAT == 1 || (shared ? p.sh_merged : p.merged)) ? 1u : NMAT;
                if (ENC == kEncPlanar) {
                    // the (d, dmin) pairs of the item's rows over the whole K: RM * nblk * 4 bytes per matrix = lines of 256 bytes
                    ok = gwait(&dempty[ds], dph ^ 1u);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&dfull[ds], NMAT * p.dm_mat_bytes);
                    for (uint32_t m = 0; m < ncopy; ++m)
                        tma_load_4d_g(gsm + p.off_d + ds * p.d_stage_bytes + m * p.dm_mat_bytes, &maps.d[mi + ms * m], 0,
                                      static_cast<int>(rb * (p.dm_mat_bytes / 256u)), 0, el, &dfull[ds]);
                    if (++ds == 2) { ds = 0; dph ^= 1u; }
                }
                for (uint32_t sb = 0; sb < p.nblk && ok; ++sb) {
                    // quant stage: code lines [matrix][RM][128 B], then factor bytes [matrix][RM][16 B]
                    ok = gwait(&qempty[qs], qph ^ 1u);
                    if (!ok) break;
                    uint8_t* q = gsm + p.off_q + qs * p.q_stage_bytes;
                    mbar_arrive_expect_tx(&qfull[qs], kRowsM * 128u + kRowsM * 16u);
                    if (Q8) {
                        // four blocks of every row: [matrix][RM][144 B]; odd spans start 8 bytes early (16-byte aligned x)
                        const int x = static_cast<int>(sb * 136u - ((sb & 1u) ? 8u : 0u));
                        for (uint32_t m = 0; m < ncopy; ++m)
                            tma_load_4d_g(q + m * (RM * 144u), &maps.q[mi + ms * m], x, r0, 0, el, &qfull[qs]);
                    } else
                    for (uint32_t m = 0; m < ncopy; ++m) {
                        tma_load_5d_g(q + m * (RM * 128u), &maps.q[mi + ms * m], 0, r0, static_cast<int>(sb), 0, el, &qfull[qs]);
                        if (GGUF) tma_load_5d_g(q + kRowsM * 128u + m * (RM * 16u), &maps.f[mi + ms * m], 0, r0, static_cast<int>(sb), 0, el, &qfull[qs]);
                        else tma_load_4d_g(q + kRowsM * 128u + m * (RM * 16u), &maps.f[mi + ms * m], static_cast<int>(sb * 16), r0, 0, el, &qfull[qs]);
                    }
                    if (++qs == 2) { qs = 0; qph ^= 1u; }
                }
            }
            if (!ok) raise_error(p.error, TSP_ERR_TIMEOUT);
        }
    } else if (warp == 2 + kDqWarps) {
        // =========================== activation-tile producer ===========================
        bool ok = true;
        uint32_t st = 0, sph = 0;   // stage of the next chunk and its phase
        for (;;) {
            const SchedItem it = sched.next(lane);
            if (it.item >= n_items) { ok = it.item != 0xffffffffu; break; }
            if (lane == 0) {
                const GTask& t = it.t;
                const bool shared = t.expert >= p.experts;
                const uint32_t nsub = sub_tiles(t);
                const uint32_t nc0 = sub_cols(sub_count(t, 0)), nc1 = sub_cols(sub_count(t, 1));
                const CUtensorMap* map0 = &maps.x[(shared ? 3 : 0) + (nc0 == 32 ? 0 : (nc0 == 64 ? 1 : 2))];
                const CUtensorMap* map1 = &maps.x[(shared ? 3 : 0) + (nc1 == 32 ? 0 : (nc1 == 64 ? 1 : 2))];
                const uint32_t bytes = (nc0 + (nsub > 1 ? nc1 : 0u)) * 128u;
                for (uint32_t c = 0; c < chunks_per_item && ok; ++c) {
                    ok = gwait(&empty[st], sph ^ 1u);
                    if (!ok) break;
                    uint8_t* b0 = stages + st * kStageBytes + 16384u;
                    mbar_arrive_expect_tx(&full[st], bytes);
                    // byte coordinate: the map's element is a byte
                    tma_load_2d(b0, map0, static_cast<int>(c * 128), static_cast<int>(t.row0), &full[st]);
                    if (nsub > 1) tma_load_2d(b0 + 16384u, map1, static_cast<int>(c * 128), static_cast<int>(t.row0 + kSub), &full[st]);
                    if (++st == kStages) { st = 0; sph ^= 1u; }
                }
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            st = __shfl_sync(0xffffffffu, st, 0); sph = __shfl_sync(0xffffffffu, sph, 0);
        }
        if (!ok && lane == 0) raise_error(p.error, TSP_ERR_TIMEOUT);
    } else if (warp == 1) {
        // =========================== MMA issuer ===========================
        bool ok = true;
        uint32_t st = 0, sph = 0, ab = 0, accph = 0;
        for (;;) {
            const SchedItem it = sched.next(lane);
            if (it.item >= n_items) { ok = it.item != 0xffffffffu; break; }
            if (lane == 0) {
                const GTask& t = it.t;
                const uint32_t nsub = sub_tiles(t);
                const uint32_t nc0 = sub_cols(sub_count(t, 0)), nc1 = sub_cols(sub_count(t, 1));
                const bool wide = nsub > 1 && nc1 == kSub;          // both sub-tiles full: one N = 256 instruction over the adjacent tiles
                const uint32_t id0 = umma_idesc_f16(kRowsM, wide ? 256u : nc0), id1 = umma_idesc_f16(kRowsM, nc1);
                const uint32_t dcol = tmem_base + ab * 256u;
                ok = gwait(&acc_empty[ab], accph ^ 1u);   // the epilogue has drained this accumulator set (used two items ago)
                if (ok) tc_fence_after();
                for (uint32_t c = 0; c < chunks_per_item && ok; ++c) {
                    ok = gwait(&full[st], sph);
                    if (!ok) break;
                    tc_fence_after();
                    const uint8_t* sbase = stages + st * kStageBytes;
                    const uint64_t adesc = umma_desc_k128(sbase), bdesc = umma_desc_k128(sbase + 16384u);
#pragma unroll
                    for (uint32_t kk = 0; kk < 4; ++kk) umma_f16(dcol, adesc + kk * 2, bdesc + kk * 2, id0, (c | kk) != 0 ? 1u : 0u);
                    if (nsub > 1 && !wide) {
                        const uint64_t bdesc1 = umma_desc_k128(sbase + 32768u);
#pragma unroll
                        for (uint32_t kk = 0; kk < 4; ++kk) umma_f16(dcol + kSub, adesc + kk * 2, bdesc1 + kk * 2, id1, (c | kk) != 0 ? 1u : 0u);
                    }
                    umma_commit(&empty[st]);   // the stage is free once the MMAs above have read it
                    if (++st == kStages) { st = 0; sph ^= 1u; }
                }
                if (ok) umma_commit(&acc_full[ab]);
                if (++ab == 2) { ab = 0; accph ^= 1u; }
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            st = __shfl_sync(0xffffffffu, st, 0); sph = __shfl_sync(0xffffffffu, sph, 0);
            ab = __shfl_sync(0xffffffffu, ab, 0); accph = __shfl_sync(0xffffffffu, accph, 0);
        }
        if (!ok && lane == 0) raise_error(p.error, TSP_ERR_TIMEOUT);
    } else if (warp < 2 + kDqWarps) {
        // =========================== dequantise (warps 2 .. 2 + kDqWarps - 1) ===========================
        const uint32_t dt = threadIdx.x - 64;                 // 0..255
        const uint32_t half = dt >> 7;                        // which K chunks of every super-block: half, half + 2
        const uint32_t r = dt & 127u;                         // A row of the item
        // the row's line in the quant stage: gate-up interleaves 16 gate + 16 up rows per lane quarter
        const uint32_t mat = GATEUP ? ((r >> 4) & 1u) : 0u;
        const uint32_t mrow = GATEUP ? ((r >> 5) * 16u + (r & 15u)) : r;          // row inside the matrix's RM rows
        const uint32_t line = mat * RM + mrow;
        const uint32_t sw = r & 7u;                           // == line & 7
        bool ok = true;
        uint32_t qs = 0, qph = 0, ds = 0, dph = 0;
        // this thread's chunks are every other one of the launch-wide chunk sequence: its stage advances by two (mod kStages)
        uint32_t st = half % kStages, sph = 0;
        for (;;) {
            const SchedItem it = sched.next(lane);
            if (it.item >= n_items) { ok = it.item != 0xffffffffu; break; }
            if (ENC == kEncPlanar && ok) ok = gwait(&dfull[ds], dph);
            const uint8_t* dmp = gsm + p.off_d + ds * p.d_stage_bytes + mat * p.dm_mat_bytes + mrow * p.nblk * 4u;
            for (uint32_t sb = 0; sb < p.nblk; ++sb) {
                if (ok) ok = gwait(&qfull[qs], qph);
                const uint8_t* q = gsm + p.off_q + qs * p.q_stage_bytes;
                if (Q8) {
                    // this thread's chunk of the span: blocks 2 * half, 2 * half + 1 of the row's four
                    if (ok) ok = gwait(&empty[st], sph ^ 1u);
                    if (ok) {
                        const uint4* src = reinterpret_cast<const uint4*>(q + line * 144u) + half * 4u;
                        uint32_t L[20];
#pragma unroll
                        for (int i = 0; i < 5; ++i) { const uint4 v = src[i]; L[4 * i] = v.x; L[4 * i + 1] = v.y; L[4 * i + 2] = v.z; L[4 * i + 3] = v.w; }
                        uint8_t* arow = stages + st * kStageBytes + r * 128u;
                        bool finite;
                        // first word of the chunk among the 20: byte (8 if the span is odd) + 68 * half - 64 * half
                        switch (half + 2u * (sb & 1u)) {
                            case 0: finite = q8_chunk_row<0>(L, arow, sw); break;
                            case 1: finite = q8_chunk_row<1>(L, arow, sw); break;
                            case 2: finite = q8_chunk_row<2>(L, arow, sw); break;
                            default: finite = q8_chunk_row<3>(L, arow, sw); break;
                        }
                        if (!finite) raise_error(p.error, TSP_ERR_NONFINITE);
                        fence_async_smem();
                    }
                    __syncwarp();
                    if (lane == 0 && ok) mbar_arrive(&full[st]);
                    st += 2;
                    if (st >= kStages) { st -= kStages; sph ^= 1u; }
                    __syncwarp();
                    if (lane == 0 && ok) mbar_arrive(&qempty[qs]);
                    if (++qs == 2) { qs = 0; qph ^= 1u; }
                    continue;
                }
                // d, dmin and the sixteen 6-bit factors of this row's super-block
                uint4 fac = *reinterpret_cast<const uint4*>(q + kRowsM * 128u + line * 16u);
                uint32_t dmw;
                if (GGUF) {
                    // header word 0 = (d, dmin); bytes 4..15 hold the low 6 bits of factors 0..3 with the top 2 bits of factors
                    // 4..7 above them (scales, then minima), then the low 4 bits of scales / minima 4..7 as nibble pairs
                    dmw = fac.x;
                    const uint32_t s_lo = fac.y & 0x3f3f3f3fu, m_lo = fac.z & 0x3f3f3f3fu;
                    const uint32_t s_hi = (fac.w & 0x0f0f0f0fu) | ((fac.y >> 2) & 0x30303030u);
                    const uint32_t m_hi = ((fac.w >> 4) & 0x0f0f0f0fu) | ((fac.z >> 2) & 0x30303030u);
                    fac = make_uint4(s_lo, s_hi, m_lo, m_hi);
                } else {
                    dmw = *reinterpret_cast<const uint32_t*>(dmp + sb * 4u);
                }
                const float dd = half_bits_to_float(dmw & 0xffffu), dmn = half_bits_to_float(dmw >> 16);
                if (ok && (!finite_f32(dd) || !finite_f32(dmn))) raise_error(p.error, TSP_ERR_NONFINITE);
                const uint8_t* codes = q + line * 128u;
#pragma unroll
                for (uint32_t pp = 0; pp < 2; ++pp) {
                    const uint32_t c = 2 * pp + half;          // chunk of the super-block
                    if (ok) ok = gwait(&empty[st], sph ^ 1u);  // the MMAs that read this stage kStages chunks ago are done
                    if (ok) {
                        const ChunkScale cs = chunk_scale(dd, dmn, pp ? fac.y : fac.x, pp ? fac.w : fac.z, 2u * half);
                        const uint4 w0 = *reinterpret_cast<const uint4*>(codes + (((2 * c) ^ sw) << 4));
                        const uint4 w1 = *reinterpret_cast<const uint4*>(codes + (((2 * c + 1) ^ sw) << 4));
                        uint8_t* arow = stages + st * kStageBytes + r * 128u;
                        uint4 lo, hi;
                        dequant8(w0.x, w0.y, cs, lo, hi);
                        *reinterpret_cast<uint4*>(arow + ((0u ^ sw) << 4)) = lo; *reinterpret_cast<uint4*>(arow + ((4u ^ sw) << 4)) = hi;
                        dequant8(w0.z, w0.w, cs, lo, hi);
                        *reinterpret_cast<uint4*>(arow + ((1u ^ sw) << 4)) = lo; *reinterpret_cast<uint4*>(arow + ((5u ^ sw) << 4)) = hi;
                        dequant8(w1.x, w1.y, cs, lo, hi);
                        *reinterpret_cast<uint4*>(arow + ((2u ^ sw) << 4)) = lo; *reinterpret_cast<uint4*>(arow + ((6u ^ sw) << 4)) = hi;
                        dequant8(w1.z, w1.w, cs, lo, hi);
                        *reinterpret_cast<uint4*>(arow + ((3u ^ sw) << 4)) = lo; *reinterpret_cast<uint4*>(arow + ((7u ^ sw) << 4)) = hi;
                        fence_async_smem();   // make the generic-proxy writes visible to the tensor-core (async) proxy
                    }
                    __syncwarp();
                    if (lane == 0 && ok) mbar_arrive(&full[st]);
                    st += 2;
                    if (st >= kStages) { st -= kStages; sph ^= 1u; }
                }
                __syncwarp();
                if (lane == 0 && ok) mbar_arrive(&qempty[qs]);
                if (++qs == 2) { qs = 0; qph ^= 1u; }
            }
            if (ENC == kEncPlanar) {
                __syncwarp();
                if (lane == 0 && ok) mbar_arrive(&dempty[ds]);
                if (++ds == 2) { ds = 0; dph ^= 1u; }
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
        }
        if (!ok && lane == 0) raise_error(p.error, TSP_ERR_TIMEOUT);
    } else {
        // =========================== epilogue (the last kEpWarps warps) ===========================
        const uint32_t quarter = warp & 3u;                   // tensor-memory lane quarter this warp may read
        const uint32_t ehalf = (warp - (3 + kDqWarps)) >> 2;  // the two warps of a quarter take the 32-column batches in turn
        uint8_t* const etile = gsm + p.off_ep + (warp - (3 + kDqWarps)) * kEpTileBytes;   // this warp's transposition tile
        bool ok = true;
        uint32_t ab = 0, accph = 0;
        for (;;) {
            const SchedItem it = sched.next(lane);
            if (it.item >= n_items) { ok = it.item != 0xffffffffu; break; }
            const GTask& t = it.t;
            const uint32_t rb = it.item % p.row_blocks;
            const bool shared = t.expert >= p.experts;
            const uint32_t nsub = sub_tiles(t);
            // down: route ids of this lane's columns (column j0 + lane of each batch), fetched before the wait so their latency
            // hides behind the MMAs: slot [g][b] = batch j0 = ehalf * 32 + 64 * b of sub-tile g
            uint32_t rt[2][2] = {{0, 0}, {0, 0}};
            if (!GATEUP) {
#pragma unroll
                for (uint32_t g = 0; g < 2; ++g)
#pragma unroll
                    for (uint32_t b = 0; b < 2; ++b) {
                        const uint32_t j = ehalf * 32 + 64 * b + lane;
                        if (j < sub_count(t, g)) {
                            const uint32_t at = t.start + g * kSub + j;
                            rt[g][b] = shared ? at : p.token_map[static_cast<uint64_t>(t.expert) * p.tokens + at];
                        }
                    }
            }
            ok = gwait(&acc_full[ab], accph);
            if (ok) {
                tc_fence_after();
                char* const obase = reinterpret_cast<char*>(shared ? p.sh_out : p.out);
                const uint64_t ostride = shared ? p.sh_out_stride_bytes : p.out_stride_bytes;
                bool bad = false;
#pragma unroll
                for (uint32_t g = 0; g < 2; ++g) {
                    if (g >= nsub) break;
                    const uint32_t cnt = sub_count(t, g), nc = sub_cols(cnt);
                    const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + ab * 256u + g * kSub;
#pragma unroll
                    for (uint32_t b = 0; b < 2; ++b) {
                        const uint32_t j0 = ehalf * 32 + 64 * b;
                        if (j0 >= nc || j0 >= cnt) break;
                        uint32_t v[32];
                        tmem_ld32(taddr + j0, v);
                        tmem_ld_wait();
                        // Results leave through a per-warp transposition tile in shared memory: the accumulators arrive with a lane per
                        // weight row and a register per token column, the output rows want a lane per token and a run of weight rows
                        // (16-byte stores instead of one 2-byte store per value).
                        if constexpr (GATEUP) {
                            // lanes 0..15 hold the gate rows of 16 hidden units, lanes 16..31 the up rows of the same units. For each
                            // pair of token columns the low half-warp finishes the even column and the high half-warp the odd one.
                            // hidden rows feed the down GEMM as its K operand: same order inside each run of 8 as the weight tiles use
                            const uint32_t u16 = lane & 15u;
                            const uint32_t hpos = (u16 & 8u) | ((u16 & 4u) | ((u16 & 1u) << 1) | ((u16 & 2u) >> 1));
                            const bool low = lane < 16;
                            constexpr uint32_t RS = 48;   // tile row: 16 units x 2 B, padded so that the 16-byte reads below spread over the banks
#pragma unroll
                            for (uint32_t a = 0; a < 16; ++a) {
                                const uint32_t send = low ? v[2 * a + 1] : v[2 * a];
                                const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, 16);
                                const float gv = __uint_as_float(low ? v[2 * a] : recv);
                                const float uv = __uint_as_float(low ? recv : v[2 * a + 1]);
                                const float val = __fdividef(gv, 1.f + __expf(-gv)) * uv;   // silu(g) * u
                                const __half hv = __float2half_rn(val);
                                const uint32_t i = 2 * a + (low ? 0u : 1u);
                                bad |= (j0 + i < cnt) && !finite_f32(__half2float(hv));
                                *reinterpret_cast<__half*>(etile + i * RS + hpos * 2) = hv;
                            }
                            __syncwarp();
                            if (j0 + lane < cnt) {   // this lane's token: 16 hidden units = 32 bytes
                                const uint4 o0 = *reinterpret_cast<const uint4*>(etile + lane * RS), o1 = *reinterpret_cast<const uint4*>(etile + lane * RS + 16);
                                uint4* dst = reinterpret_cast<uint4*>(obase + static_cast<uint64_t>(t.row0 + g * kSub + j0 + lane) * ostride + (rb * 64u + quarter * 16u) * 2);
                                dst[0] = o0; dst[1] = o1;
                            }
                            __syncwarp();
                        } else {
                            const uint32_t wbase = rb * kRowsM + quarter * 32;   // first output channel of this warp
                            const bool f16 = !shared && p.out_f16;
                            bool nf = false;
#pragma unroll
                            for (uint32_t i = 0; i < 32; ++i) nf |= (j0 + i < cnt) && !finite_f32(__uint_as_float(v[i]));
                            bad |= nf;
                            char* orow = obase + static_cast<uint64_t>(rt[g][b]) * ostride;   // this lane's token = column j0 + lane
                            if (f16) {
                                constexpr uint32_t RS = 80;   // 32 channels x 2 B + 16
#pragma unroll
                                for (uint32_t i = 0; i < 32; ++i) *reinterpret_cast<__half*>(etile + i * RS + lane * 2) = __float2half_rn(__uint_as_float(v[i]));
                                __syncwarp();
                                if (j0 + lane < cnt) {
                                    uint4* dst = reinterpret_cast<uint4*>(orow + wbase * 2);
#pragma unroll
                                    for (uint32_t k = 0; k < 4; ++k) dst[k] = *reinterpret_cast<const uint4*>(etile + lane * RS + k * 16);
                                }
                            } else {
                                constexpr uint32_t RS = 144;  // 32 channels x 4 B + 16
#pragma unroll
                                for (uint32_t i = 0; i < 32; ++i) *reinterpret_cast<uint32_t*>(etile + i * RS + lane * 4) = v[i];
                                __syncwarp();
                                if (j0 + lane < cnt) {
                                    uint4* dst = reinterpret_cast<uint4*>(orow + wbase * 4);
#pragma unroll
                                    for (uint32_t k = 0; k < 8; ++k) dst[k] = *reinterpret_cast<const uint4*>(etile + lane * RS + k * 16);
                                }
                            }
                            __syncwarp();
                        }
                    }
                }
                if (bad) raise_error(p.error, TSP_ERR_NONFINITE);
                tc_fence_before();
            }
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(&acc_empty[ab]);
            if (++ab == 2) { ab = 0; accph ^= 1u; }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
        }
        if (!ok && lane == 0) raise_error(p.error, TSP_ERR_TIMEOUT);
    }
    // every path ends here: free the tensor memory
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ---------------------------------------------------------------------------------------------
// test hook: the binary16 values the GEMM kernel stages for one planar Q4_K expert, in natural K order
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) staged_f16_kernel(const uint8_t* __restrict__ expert, uint32_t rows, uint32_t nblk, __half* __restrict__ out) {
    const uint32_t row = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const uint64_t units = static_cast<uint64_t>(rows) * nblk;
    for (uint32_t u = threadIdx.x & 31u; u < nblk * 4; u += 32) {   // (super-block, chunk) of this row
        const uint32_t sb = u >> 2, c = u & 3u;
        const uint64_t blk = static_cast<uint64_t>(row) * nblk + sb;
        const uint4 fac = *reinterpret_cast<const uint4*>(expert + units * 128 + blk * 16);
        const uint32_t dmw = *reinterpret_cast<const uint32_t*>(expert + units * 144 + blk * 4);
        const ChunkScale cs = chunk_scale(half_bits_to_float(dmw & 0xffffu), half_bits_to_float(dmw >> 16), (c & 2u) ? fac.y : fac.x,
                                          (c & 2u) ? fac.w : fac.z, 2u * (c & 1u));
        const uint32_t* codes = reinterpret_cast<const uint32_t*>(expert + blk * 128 + c * 32);
        __half* dst = out + static_cast<uint64_t>(row) * nblk * 256 + sb * 256 + c * 64;
#pragma unroll
        for (uint32_t qq = 0; qq < 4; ++qq) {
            uint4 lo, hi;
            dequant8(codes[2 * qq], codes[2 * qq + 1], cs, lo, hi);
            const uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w}, hw[4] = {hi.x, hi.y, hi.z, hi.w};
            const int pos[8] = {0, 2, 1, 3, 4, 6, 5, 7};   // stored position i holds K element pos[i] of the run
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                dst[8 * qq + pos[i]] = __ushort_as_half(static_cast<unsigned short>((lw[i >> 1] >> (16 * (i & 1))) & 0xffffu));
                dst[32 + 8 * qq + pos[i]] = __ushort_as_half(static_cast<unsigned short>((hw[i >> 1] >> (16 * (i & 1))) & 0xffffu));
            }
        }
    }
}

int launch_staged_f16(const uint8_t* expert, uint32_t rows, uint32_t cols, void* out, cudaStream_t st) {
    staged_f16_kernel<<<(rows + 3) / 4, 128, 0, st>>>(expert, rows, cols / 256, static_cast<__half*>(out));
    TSP_CUDA(cudaGetLastError());
    return TSP_OK;
}

// ---------------------------------------------------------------------------------------------
// helpers: route offsets, the K-ordered binary16 copy of the input rows
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) route_offsets_kernel(const uint32_t* __restrict__ counts, uint32_t experts, uint32_t* __restrict__ offsets) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ uint32_t warp_sum[8];
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t carry = 0;
    for (uint32_t base = 0; base < experts; base += 256) {
        const uint32_t e = base + tid;
        const uint32_t c = e < experts ? counts[e] : 0u;
        uint32_t incl = c;
        for (int o = 1; o < 32; o <<= 1) { const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= static_cast<uint32_t>(o)) incl += v; }
        if (lane == 31) warp_sum[warp] = incl;
        __syncthreads();
        uint32_t before = 0, total = 0;
        for (uint32_t i = 0; i < 8; ++i) { if (i < warp) before += warp_sum[i]; total += warp_sum[i]; }
        if (e < experts) offsets[e] = carry + before + incl - c;
        carry += total;
        __syncthreads();
    }
    if (tid == 0) {
        offsets[experts] = carry;
        offsets[experts + 1] = 0;   // the item counters of the grouped GEMM launches that follow (routed gate-up, routed down, and
        offsets[experts + 2] = 0;   // the two dense launches of a shared expert in another encoding)
        offsets[experts + 3] = 0;
        offsets[experts + 4] = 0;
    }
}

// Rows (FP32 or binary16) -> binary16 rows with the K order 0,2,1,3,4,6,5,7 inside each run of 8: the B operand of the
// gate-up GEMM, fetched from here by token id. 64 threads per row, four rows per CTA.
template <bool IN16>
__global__ void __launch_bounds__(256)
rows_f16k_kernel(const void* __restrict__ x, uint64_t x_stride, uint32_t rows, uint32_t cols, __half* __restrict__ xk, uint64_t xk_stride, uint32_t* error) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t row = blockIdx.x * 4 + (threadIdx.x >> 6);
    if (row >= rows) return;
    const uint32_t t64 = threadIdx.x & 63;
    const char* src = reinterpret_cast<const char*>(x) + static_cast<uint64_t>(row) * x_stride;
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(xk) + static_cast<uint64_t>(row) * xk_stride);
    bool bad = false;
    for (uint32_t k8 = t64; k8 < cols / 8; k8 += 64) {
        uint32_t h[8];
        if (IN16) {
            const uint4 v = reinterpret_cast<const uint4*>(src)[k8];
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                h[2 * i] = w[i] & 0xffffu; h[2 * i + 1] = w[i] >> 16;
                bad |= (w[i] & 0x7c00u) == 0x7c00u || (w[i] & 0x7c000000u) == 0x7c000000u;
            }
        } else {
            const float4 a = reinterpret_cast<const float4*>(src)[2 * k8], b = reinterpret_cast<const float4*>(src)[2 * k8 + 1];
            const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) { const __half hv = __float2half_rn(v[i]); bad |= !finite_f32(__half2float(hv)); h[i] = __half_as_ushort(hv); }
        }
        dst[k8] = make_uint4(h[0] | (h[2] << 16), h[1] | (h[3] << 16), h[4] | (h[6] << 16), h[5] | (h[7] << 16));
    }
    if (bad) raise_error(error, TSP_ERR_NONFINITE);
}

// Routed copy of the K-ordered input rows: position p of the permuted order belongs to the expert e with
// offsets[e] <= p < offsets[e+1]; its route id is token_map[e*tokens + p - offsets[e]], its input row route / selected.
__global__ void __launch_bounds__(256)
gather_rows16_kernel(const uint4* __restrict__ xk, uint64_t xk_stride, const uint32_t* __restrict__ token_map, const uint32_t* __restrict__ offsets,
                     uint32_t experts, uint32_t tokens, uint32_t selected, uint32_t cols, uint4* __restrict__ xp, uint64_t xp_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t pos = blockIdx.x * 4 + (threadIdx.x >> 6);
    if (pos >= offsets[experts]) return;
    uint32_t lo = 0, hi = experts;   // largest e with offsets[e] <= pos
    while (hi - lo > 1) { const uint32_t mid = (lo + hi) >> 1; if (offsets[mid] <= pos) lo = mid; else hi = mid; }
    const uint32_t row = token_map[static_cast<uint64_t>(lo) * tokens + (pos - offsets[lo])] / selected;
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(xk) + static_cast<uint64_t>(row) * xk_stride);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(xp) + static_cast<uint64_t>(pos) * xp_stride);
    for (uint32_t k8 = threadIdx.x & 63u; k8 < cols / 8; k8 += 64) dst[k8] = src[k8];
}

int launch_gather_rows16(const void* xk, uint64_t xk_stride, const uint32_t* token_map, const uint32_t* offsets, uint32_t experts, uint32_t tokens,
                         uint32_t selected, uint32_t cols, void* xp, uint64_t xp_stride, cudaStream_t st) {
    const uint32_t routes = tokens * selected;
    TSP_CUDA(launch_pdl(gather_rows16_kernel, dim3((routes + 3) / 4), dim3(256), 0, st, static_cast<const uint4*>(xk), xk_stride, token_map, offsets,
                        experts, tokens, selected, cols, static_cast<uint4*>(xp), xp_stride));
    return TSP_OK;
}

int launch_route_offsets(const uint32_t* counts, uint32_t experts, uint32_t* offsets, cudaStream_t st) {
    TSP_CUDA(launch_pdl(route_offsets_kernel, dim3(1), dim3(256), 0, st, counts, experts, offsets));
    return TSP_OK;
}

int launch_rows_f16k(const void* x, uint64_t x_stride, uint32_t x_dtype, uint32_t rows, uint32_t cols, void* xk, uint64_t xk_stride, uint32_t* error,
                     cudaStream_t st) {
    if (x_dtype == 1)
        TSP_CUDA(launch_pdl(rows_f16k_kernel<true>, dim3((rows + 3) / 4), dim3(256), 0, st, x, x_stride, rows, cols, static_cast<__half*>(xk), xk_stride, error));
    else
        TSP_CUDA(launch_pdl(rows_f16k_kernel<false>, dim3((rows + 3) / 4), dim3(256), 0, st, x, x_stride, rows, cols, static_cast<__half*>(xk), xk_stride, error));
    return TSP_OK;
}

// ---------------------------------------------------------------------------------------------
// host launcher of the grouped tensor-core GEMMs
// ---------------------------------------------------------------------------------------------
template <bool GATEUP, int ENC>
static int launch_grouped_t(const GroupedMaps& m, const GroupedParams& p, size_t smem, int grid, cudaStream_t st) {
    auto kernel = grouped_mma_kernel<GATEUP, ENC>;
    static thread_local SmemAttrCache configured;   // per kernel instantiation, keyed by device
    TSP_CUDA(ensure_dynamic_smem(kernel, configured, smem));
    TSP_CUDA(launch_pdl(kernel, dim3(grid), dim3(kGWarps * 32), smem, st, m, p));
    return TSP_OK;
}

// a/b: Q4_K matrix sets [rows x cols], Pack v3 planar or plain GGUF super-blocks, or Q8_0 GGUF blocks (both sets and the shared
// expert's in the same encoding and layout). tasks == nullptr: a dense launch, only the shared expert's rows (`sh`) are computed
// and a/b only give the shape.
// gate-up: act = the routed copy of the K-ordered input rows in permuted position order (act_rows of them);
//          out = binary16 hidden rows [positions x rows] in permuted position order; shared expert: sh->act = the K-ordered
//          input rows by token, sh->out hidden rows by token.
// down:    act = hidden rows in permuted position order (act_rows of them); out = route rows by route id, FP32 or binary16;
//          shared expert: sh->act hidden rows by token, sh->out FP32 rows by token.
int launch_grouped(const tsp_matrix_set* a, const tsp_matrix_set* b, bool gateup, const void* act, uint64_t act_stride, uint32_t act_rows,
                   uint32_t tokens, uint32_t selected, const uint32_t* token_map, const uint32_t* tasks, const uint32_t* counts,
                   const uint32_t* offsets, uint32_t* work_counter, void* out, uint64_t out_stride, uint32_t out_f16, uint32_t* error, cudaStream_t st,
                   const GroupedShared* sh) {
    const bool q8 = a->type == TSP_TYPE_Q8_0;
    if (a->type != TSP_TYPE_Q4_K && !(q8 && a->layout == TSP_LAYOUT_GGUF))
        return fail(TSP_E_TYPE, "grouped GEMM: the tensor-core kernel reads Q4_K (planar or GGUF blocks) and Q8_0 GGUF blocks");
    TSP_REQUIRE(tasks || sh, "grouped GEMM: a launch without a task table needs the dense rows");
    const bool gguf = a->layout == TSP_LAYOUT_GGUF;
    const uint32_t rm = gateup ? 64u : 128u;
    TSP_REQUIRE(a->rows % rm == 0 && a->cols % 256 == 0, "grouped GEMM: rows must be a multiple of %u and columns of 256", rm);
    GroupedParams p{};
    const uint32_t nblk = q8 ? a->cols / 128 : a->cols / 256;
    TSP_REQUIRE(a->cols / 256 <= 32, "grouped GEMM: K extent too large");
    p.split = a->split < a->experts ? a->split : a->experts;
    p.experts = a->experts;
    p.nblk = nblk; p.chunks = a->cols / 64; p.row_blocks = a->rows / rm;
    const uint64_t total_units = static_cast<uint64_t>(a->rows) * nblk;
    const uint64_t sm_off = total_units * 128, dm_off = total_units * 144;
    const uint8_t* base[4] = {static_cast<const uint8_t*>(a->base), static_cast<const uint8_t*>(a->base_hi ? a->base_hi : a->base), nullptr, nullptr};
    if (gateup) {
        base[2] = static_cast<const uint8_t*>(b->base);
        base[3] = static_cast<const uint8_t*>(b->base_hi ? b->base_hi : b->base);
    }
    for (int i = 0; i < (gateup ? 4 : 2); ++i) TSP_REQUIRE(reinterpret_cast<uintptr_t>(base[i]) % 16 == 0, "grouped GEMM: expert images must be 16-byte aligned");
    p.tokens = tokens; p.selected = selected; p.token_map = token_map;
    p.tasks = tasks; p.counts = counts; p.offsets = offsets;
    p.out = out; p.out_stride_bytes = out_stride; p.out_f16 = out_f16; p.error = error; p.work_counter = work_counter;
    const uint32_t nmat = gateup ? 2 : 1;
    p.dm_mat_bytes = q8 ? 0u : rm * nblk * 4u;        // a multiple of 256: rm >= 64 (Q8_0: no (d, dmin) ring)
    p.off_q = 1024;
    p.q_stage_bytes = kRowsM * (128u + 16u);
    p.off_d = p.off_q + 2 * p.q_stage_bytes;
    p.d_stage_bytes = (nmat * p.dm_mat_bytes + 1023u) & ~1023u;
    p.off_st = p.off_d + 2 * p.d_stage_bytes;
    p.off_ep = p.off_st + kStages * kStageBytes;
    const size_t smem = p.off_ep + kEpWarps * kEpTileBytes + 1024;
    TSP_REQUIRE(smem <= 227 * 1024, "grouped GEMM: K extent needs more shared memory than one SM has");

    // gate and up of an expert at one constant distance: one copy per plane brings both
    auto mergeable = [](const uint8_t* first, const uint8_t* second, uint64_t* delta) {
        if (second <= first) return false;
        *delta = static_cast<uint64_t>(second - first);
        return *delta % 16 == 0 && *delta < (1ull << 40);
    };
    uint64_t delta = 0, delta_hi = 0;
    p.merged = gateup && mergeable(base[0], base[2], &delta) && mergeable(base[1], base[3], &delta_hi) && delta == delta_hi;
    GroupedMaps maps;
    auto plane_maps = [&](const uint8_t* bp, uint32_t mats, uint64_t ds, uint32_t n, uint64_t stride, uint32_t at) -> int {
        if (q8) {
            // rows of 34-byte blocks: [row bytes][row][matrix][expert]; a box is 144 bytes (four blocks + 8) of rm rows. Columns are a
            // multiple of 256, so a row holds an even number of spans and the last one is odd: its box (from 8 bytes before the span)
            // ends exactly at the end of the row, and every even span's box ends inside it
            const uint64_t row_bytes = uint64_t(a->cols / 32) * 34;   // a multiple of 16: columns are a multiple of 256
            const uint64_t dims[4] = {row_bytes, a->rows, mats, n}, strides[3] = {row_bytes, ds, stride};
            const uint32_t box[4] = {144, rm, mats, 1};
            if (int rc = get_tensor_map_bytes(bp, 4, dims, strides, box, false, &maps.q[at])) return rc;
            maps.f[at] = maps.q[at]; maps.d[at] = maps.q[at];   // not read
            return TSP_OK;
        }
        if (gguf) {
            // codes: bytes 16..143 of every 144-byte super-block, [128 B][row][super-block][matrix][expert], 128-byte swizzle;
            // headers: bytes 0..15 of the same blocks, same walk
            const uint64_t dims[5] = {128, a->rows, nblk, mats, n}, strides[4] = {uint64_t(nblk) * 144, 144, ds, stride};
            const uint32_t box[5] = {128, rm, 1, mats, 1};
            if (int rc = get_tensor_map_bytes(bp + 16, 5, dims, strides, box, true, &maps.q[at])) return rc;
            const uint64_t hdims[5] = {16, a->rows, nblk, mats, n};
            const uint32_t hbox[5] = {16, rm, 1, mats, 1};
            if (int rc = get_tensor_map_bytes(bp, 5, hdims, strides, hbox, false, &maps.f[at])) return rc;
            maps.d[at] = maps.f[at];   // not read
            return TSP_OK;
        }
        {   // codes: [128 B of a super-block][row][super-block][matrix][expert], 128-byte swizzle
            const uint64_t dims[5] = {128, a->rows, nblk, mats, n}, strides[4] = {uint64_t(nblk) * 128, 128, ds, stride};
            const uint32_t box[5] = {128, rm, 1, mats, 1};
            if (int rc = get_tensor_map_bytes(bp, 5, dims, strides, box, true, &maps.q[at])) return rc;
        }
        {   // factors: [16 B x super-blocks][row][matrix][expert]
            const uint64_t dims[4] = {uint64_t(nblk) * 16, a->rows, mats, n}, strides[3] = {uint64_t(nblk) * 16, ds, stride};
            const uint32_t box[4] = {16, rm, mats, 1};
            if (int rc = get_tensor_map_bytes(bp + sm_off, 4, dims, strides, box, false, &maps.f[at])) return rc;
        }
        {   // (d, dmin) pairs: the plane in lines of 256 bytes, [256 B][line][matrix][expert]; an item's rows are dm_mat_bytes / 256 lines
            const uint64_t dims[4] = {256, total_units * 4 / 256, mats, n}, strides[3] = {256, ds, stride};
            const uint32_t box[4] = {256, p.dm_mat_bytes / 256u, mats, 1};
            if (int rc = get_tensor_map_bytes(bp + dm_off, 4, dims, strides, box, false, &maps.d[at])) return rc;
        }
        return TSP_OK;
    };
    const uint32_t mats = p.merged ? 2 : 1;
    const uint64_t ds = p.merged ? delta : 16;
    const uint64_t stride = a->experts > 1 ? a->expert_stride : 16;
    TSP_REQUIRE(stride % 16 == 0, "grouped GEMM: expert stride must be a multiple of 16");
    TSP_REQUIRE(gguf || q8 || total_units * 4 % 256 == 0, "grouped GEMM: the (d, dmin) plane must be a whole number of 256-byte lines");
    const uint32_t n_lo = p.split, n_hi = a->experts - p.split;
    for (uint32_t i = 0; i < 4; ++i) {
        const uint32_t m = i >> 1;
        const bool hi = i & 1;
        if (m == 1 && (!gateup || p.merged)) { maps.q[i] = maps.q[i - 2]; maps.f[i] = maps.f[i - 2]; maps.d[i] = maps.d[i - 2]; continue; }
        if (hi && n_hi == 0) { maps.q[i] = maps.q[i - 1]; maps.f[i] = maps.f[i - 1]; maps.d[i] = maps.d[i - 1]; continue; }
        if (int rc = plane_maps(base[i], mats, ds, hi ? n_hi : (n_lo ? n_lo : 1), stride, i)) return rc;
    }
    for (int i = 4; i < 6; ++i) { maps.q[i] = maps.q[0]; maps.f[i] = maps.f[0]; maps.d[i] = maps.d[0]; }
    const uint32_t ns[3] = {32, 64, 128};
    for (int i = 0; i < 3; ++i) {
        const uint64_t dims[2] = {uint64_t(a->cols) * 2, act_rows}, strides[1] = {act_stride};
        const uint32_t box[2] = {128, ns[i]};
        if (int rc = get_tensor_map_bytes(act, 2, dims, strides, box, true, &maps.x[i])) return rc;
        maps.x[3 + i] = maps.x[i];
    }
    if (sh) {   // the layer's dense shared expert: same shape, one expert, its own rows
        const uint8_t* sa = static_cast<const uint8_t*>(sh->a->base);
        const uint8_t* sb = gateup ? static_cast<const uint8_t*>(sh->b->base) : nullptr;
        TSP_REQUIRE(reinterpret_cast<uintptr_t>(sa) % 16 == 0 && reinterpret_cast<uintptr_t>(sb) % 16 == 0, "grouped GEMM: expert images must be 16-byte aligned");
        uint64_t sdelta = 0;
        p.sh_merged = gateup && mergeable(sa, sb, &sdelta);
        p.sh_tokens = sh->tokens;
        p.sh_tasks = (sh->tokens + kTaskRoutes - 1) / kTaskRoutes;
        p.sh_out = sh->out; p.sh_out_stride_bytes = sh->out_stride;
        if (int rc = plane_maps(sa, p.sh_merged ? 2 : 1, p.sh_merged ? sdelta : 16, 1, 16, 4)) return rc;
        if (gateup && !p.sh_merged) { if (int rc = plane_maps(sb, 1, 16, 1, 16, 5)) return rc; }
        for (int i = 0; i < 3; ++i) {
            const uint64_t dims[2] = {uint64_t(a->cols) * 2, sh->tokens}, strides[1] = {sh->act_stride};
            const uint32_t box[2] = {128, ns[i]};
            if (int rc = get_tensor_map_bytes(sh->act, 2, dims, strides, box, true, &maps.x[3 + i])) return rc;
        }
    }
    const int grid = sm_count();
    if (grid <= 0) return fail(TSP_E_CUDA, "no usable CUDA device");
    if (q8) return gateup ? launch_grouped_t<true, kEncQ8>(maps, p, smem, grid, st) : launch_grouped_t<false, kEncQ8>(maps, p, smem, grid, st);
    if (gguf) return gateup ? launch_grouped_t<true, kEncGguf>(maps, p, smem, grid, st) : launch_grouped_t<false, kEncGguf>(maps, p, smem, grid, st);
    return gateup ? launch_grouped_t<true, kEncPlanar>(maps, p, smem, grid, st) : launch_grouped_t<false, kEncPlanar>(maps, p, smem, grid, st);
}

}  // namespace tsp
