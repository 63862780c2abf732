/*
 * tsp_ep.h — expert-parallel form of the routed-MoE FFN layer over the GPUs of one node (libtsp_ep.so).
 *
 * No counterpart in the reference, which drives one GPU. Experts are sharded over the ranks, tokens are data-parallel by
 * source rank, and the layer is: route locally -> pack one slab per destination rank -> NCCL all-to-all (dispatch) ->
 * the owners run the same decode / prefill kernels as on one GPU over the rows they received -> per-row partial sums ->
 * NCCL all-to-all (combine) -> local mixture with the locally computed shared expert, partial sums added in ascending rank
 * order. One process per GPU; the communicator is this library's own (`ncclCommInitRank` from an id the caller distributes).
 *
 * Slabs have a fixed size, so a step needs no host synchronisation: a slab holds a count, the routing rows (local expert slot
 * and weight per route) and the token rows of the tokens that have at least one route to that rank, each token once per rank.
 * Nothing here reads a peer's memory from a kernel: received rows sit in local HBM before any kernel (or TMA load) touches them.
 *
 * Hot experts may be replicated: an expert whose placement says "every rank" is served by the token's own rank, which removes
 * its routes from the exchange and spreads its work evenly (tokens are spread evenly).
 *
 * Return values and error reporting as in tsp_moe.h (TSP_OK / negative TSP_E_*, tsp_last_error(), sticky device error word).
 */
#ifndef TSP_EP_H
#define TSP_EP_H

#include "tsp_moe.h"

#ifdef __cplusplus
extern "C" {
#endif

#define TSP_EP_ID_BYTES 128
#define TSP_EP_REPLICATED 0xffffu   /* owner value in a placement word: every rank holds the expert */

typedef struct tsp_ep_ctx tsp_ep_ctx;

/* Message of the last refused call of this library on the calling thread. Never NULL. */
const char* tsp_ep_last_error(void);

/* Rank 0 makes an id and hands it to the other ranks by any means (a store, a broadcast); every rank then creates its context
 * with its CUDA device current. */
int tsp_ep_unique_id(uint8_t* id /* TSP_EP_ID_BYTES */);
int tsp_ep_create(const uint8_t* id, int rank, int world, tsp_ep_ctx** out);
int tsp_ep_destroy(tsp_ep_ctx* ctx);

/* One layer's placement and local weights.
 * d_place[e] = (owner << 16) | slot for every global expert e: `owner` is a rank or TSP_EP_REPLICATED, `slot` the index of
 * the expert inside the owner's (for a replicated expert: every rank's) local matrix sets.
 * local: matrix sets over this rank's `local_experts` experts (gate / up / down .experts == local_experts) and the dense
 * shared expert, as for tsp_moe_layer_decode / tsp_moe_layer_prefill. */
typedef struct tsp_ep_layer {
    tsp_moe_weights local;
    uint32_t local_experts;
    const uint32_t* d_place;
} tsp_ep_layer;

/* Bytes of the caller-owned scratch buffer (device memory, 1024-byte aligned) for steps of `tokens` rows per rank. */
uint64_t tsp_ep_scratch_bytes(uint32_t tokens, uint32_t channels, uint32_t hidden, uint32_t experts, uint32_t local_experts,
                              uint32_t selected, uint32_t world, int prefill);
/* Rows one slab holds besides the token rows (its count and routing rows, rounded up to whole token rows). */
uint32_t tsp_ep_slab_header_rows(uint32_t tokens, uint32_t channels, uint32_t selected);

/* One expert-parallel layer step for this rank's `tokens` rows (the same count on every rank).
 * d_x16: binary16 rows [tokens x channels]; d_logits: FP32 [tokens x experts]; d_out16: binary16 rows [tokens x channels].
 * prefill != 0 runs the grouped tensor-core GEMMs on the owners (Q4_K Pack v3 planar weights), else the decode-size kernels.
 * All launches and both collectives are enqueued on `stream`; nothing synchronises with the host. */
int tsp_ep_moe_layer(tsp_ep_ctx* ctx, const tsp_ep_layer* layer, void* d_scratch, uint64_t scratch_bytes, const void* d_x16,
                     uint64_t x_stride_bytes, const float* d_logits, uint64_t logits_stride_bytes, uint32_t tokens,
                     uint32_t channels, uint32_t hidden, uint32_t experts, uint32_t selected, uint32_t mode, int normalize_selected,
                     int prefill, void* d_out16, uint64_t out_stride_bytes, uint32_t* d_error, void* stream);

/* Test hooks for the slab protocol, usable without a communicator: the pack half (route -> plan -> slabs for `world` ranks as
 * rank `rank`) and the unpack half (dense routing tables from `world` received slabs). Slab p of a buffer starts at
 * p * tsp_ep_slab_bytes(). */
uint64_t tsp_ep_slab_bytes(uint32_t tokens, uint32_t channels, uint32_t selected);
int tsp_ep_pack(const uint32_t* d_ids, const float* d_weights, const void* d_x16, uint64_t x_stride_bytes, const uint32_t* d_place,
                uint32_t tokens, uint32_t channels, uint32_t selected, uint32_t rank, uint32_t world, int k_ordered, int32_t* d_pos,
                void* d_slabs, void* stream);
int tsp_ep_unpack(const void* d_slabs, uint32_t tokens, uint32_t channels, uint32_t selected, uint32_t world, uint32_t* d_ids_all,
                  float* d_weights_all, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TSP_EP_H */
