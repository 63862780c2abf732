/*
 * CPU oracle for the block-quantised routed-MoE FFN path. TEST INFRASTRUCTURE ONLY:
 * the product library never links or calls this file (see tsp_oracle.h).
 *
 * Each function restates, in plain C, the algorithm of the reference's scalar CPU code;
 * the reference file:line it follows is given beside it. Weights are decoded to exact
 * doubles and every accumulation is in double, as the reference does.
 */
#include "tsp_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

static inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | ((uint16_t)p[1] << 8)); }
static inline uint32_t rd32(const uint8_t* p) { return (uint32_t)rd16(p) | ((uint32_t)rd16(p + 2) << 16); }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

int tso_block_geometry(uint32_t type, uint32_t* epb, uint32_t* bpb) {
    /* gguf.cpp:21-32 (encoding table), restricted to the encodings on this path */
    uint32_t e, b;
    switch (type) {
        case 0: e = 1; b = 4; break;
        case 1: e = 1; b = 2; break;
        case 30: e = 1; b = 2; break;
        case 7: e = 32; b = 24; break;
        case 8: e = 32; b = 34; break;
        case 12: e = 256; b = 144; break;
        case 13: e = 256; b = 176; break;
        case 14: e = 256; b = 210; break;
        case 20: e = 32; b = 18; break;
        default: return TSO_E_TYPE;
    }
    if (epb) *epb = e;
    if (bpb) *bpb = b;
    return TSO_OK;
}

/* numeric.cpp:81-91 */
float tso_binary16(uint16_t bits) {
    const uint32_t sign = (uint32_t)(bits & 0x8000u) << 16;
    uint32_t mantissa = bits & 1023u;
    const uint32_t exponent = (bits >> 10) & 31u;
    if (exponent == 31) return bits_f32(sign | 0x7f800000u | (mantissa << 13));
    if (exponent) return bits_f32(sign | ((exponent + 112) << 23) | (mantissa << 13));
    if (!mantissa) return bits_f32(sign);
    uint32_t e = 113;
    while (!(mantissa & 1024u)) { mantissa <<= 1; --e; }
    return bits_f32(sign | (e << 23) | ((mantissa & 1023u) << 13));
}

/* numeric.cpp:25-31: six-bit scale (minimum=0) or min (minimum=1) of 32-wide group `group` */
static uint32_t k_group_factor(const uint8_t* block, uint32_t group, int minimum) {
    const uint32_t lane = group & 3u;
    const uint32_t base = 4 + lane + (minimum ? 4u : 0u);
    if (group < 4) return block[base] & 63u;
    const uint32_t packed = block[12 + lane];
    const uint32_t upper = block[base] >> 6;
    return ((packed >> (minimum ? 4 : 0)) & 15u) | (upper << 4);
}

/* numeric.cpp:33-68 */
double tso_value(uint32_t type, const uint8_t* block, uint32_t index) {
    switch (type) {
        case 0: return bits_f32(rd32(block));
        case 1: return tso_binary16(rd16(block));
        case 30: return bits_f32((uint32_t)rd16(block) << 16);
        case 7: {   /* Q5_1: d, m, 32 fifth bits, 16 bytes of nibbles (numeric.cpp:38-42) */
            const uint32_t low = (block[8 + index % 16] >> (4 * (index / 16))) & 15u;
            const uint32_t high = (rd32(block + 4) >> index) & 1u;
            return (double)tso_binary16(rd16(block)) * (low | (high << 4)) + tso_binary16(rd16(block + 2));
        }
        case 8: return (double)tso_binary16(rd16(block)) * (int8_t)block[2 + index];
        case 12: case 13: {   /* Q5_K: the Q4_K header, 32 bytes of fifth bits, then the nibbles (numeric.cpp:44-50) */
            const uint32_t low_offset = type == 12 ? 16u : 48u;
            uint32_t q = (block[low_offset + (index / 64) * 32 + index % 32] >> (4 * ((index % 64) / 32))) & 15u;
            if (type == 13) q |= ((block[16 + index % 32] >> (index / 32)) & 1u) << 4;
            return (double)tso_binary16(rd16(block)) * k_group_factor(block, index / 32, 0) * q -
                   (double)tso_binary16(rd16(block + 2)) * k_group_factor(block, index / 32, 1);
        }
        case 14: {  /* Q6_K: 128 bytes of low nibbles, 64 bytes of 2-bit tops, 16 signed group scales, d (numeric.cpp:51-58) */
            const uint32_t within = index % 128, section = index / 128;
            const uint32_t low = (block[section * 64 + within % 64] >> (4 * (within / 64))) & 15u;
            const uint32_t high = (block[128 + section * 32 + within % 32] >> (2 * (within / 32))) & 3u;
            const int scale = (int8_t)block[192 + index / 16];
            return (double)tso_binary16(rd16(block + 208)) * scale * ((int)(low | (high << 4)) - 32);
        }
        case 20: {  /* IQ4_NL: d and 16 bytes of nibbles that index the encoding's fixed 16-value alphabet (numeric.cpp:59-65) */
            static const int alphabet[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
            const uint32_t code = (block[2 + index % 16] >> (4 * (index / 16))) & 15u;
            return (double)tso_binary16(rd16(block)) * alphabet[code];
        }
        default: return NAN;
    }
}

static int check_extent(uint32_t type, size_t nbytes, size_t elements, uint32_t* epb, uint32_t* bpb) {
    if (tso_block_geometry(type, epb, bpb) != TSO_OK) return TSO_E_TYPE;
    if (!elements || elements % *epb || (elements / *epb) * (size_t)*bpb != nbytes) return TSO_E_SHAPE;
    return TSO_OK;
}

/* numeric.cpp:97-148 (generic branch) */
int tso_dequantize(uint32_t type, const uint8_t* bytes, size_t nbytes, float* out, size_t elements) {
    uint32_t epb, bpb;
    const int rc = check_extent(type, nbytes, elements, &epb, &bpb);
    if (rc) return rc;
    for (size_t start = 0; start < elements; start += epb) {
        const uint8_t* block = bytes + (start / epb) * bpb;
        for (uint32_t i = 0; i < epb; ++i) {
            const double v = tso_value(type, block, i);
            if (!isfinite(v)) return TSO_E_NONFINITE;
            const float r = (float)v;
            if (!isfinite(r)) return TSO_E_NONFINITE;
            out[start + i] = r;
        }
    }
    return TSO_OK;
}

/* numeric.cpp:150-184. The inner loop decodes the block's header once; the products and
 * the order of the double additions are the reference's. */
static int gemv_core(uint32_t type, const uint8_t* matrix, size_t nbytes, uint32_t columns, uint32_t rows,
                     const double* xd, const float* xf, double* output) {
    uint32_t epb, bpb;
    if (!rows) return TSO_E_SHAPE;
    const int rc = check_extent(type, nbytes, (size_t)columns * rows, &epb, &bpb);
    if (rc) return rc;
    if (columns % epb) return TSO_E_SHAPE;
    for (uint32_t c = 0; c < columns; ++c) if (!isfinite(xd ? xd[c] : (double)xf[c])) return TSO_E_NONFINITE;
    const size_t bpr = columns / epb;
    for (uint32_t row = 0; row < rows; ++row) {
        double sum = 0;
        for (size_t g = 0; g < bpr; ++g) {
            const uint8_t* block = matrix + ((size_t)row * bpr + g) * bpb;
            const size_t x0 = g * epb;
            if (type == 12) {
                const double d = tso_binary16(rd16(block)), dmin = tso_binary16(rd16(block + 2));
                for (uint32_t grp = 0; grp < 8; ++grp) {
                    const double sc = k_group_factor(block, grp, 0), mn = k_group_factor(block, grp, 1);
                    const uint8_t* q = block + 16 + (grp / 2) * 32;
                    const uint32_t shift = 4 * (grp & 1u);
                    for (uint32_t l = 0; l < 32; ++l) {
                        const double w = d * sc * ((q[l] >> shift) & 15u) - dmin * mn;
                        if (!isfinite(w)) return TSO_E_NONFINITE;
                        const size_t k = x0 + grp * 32 + l;
                        sum += w * (xd ? xd[k] : (double)xf[k]);
                    }
                }
            } else if (type == 8) {
                const double d = tso_binary16(rd16(block));
                for (uint32_t l = 0; l < 32; ++l) {
                    const double w = d * (int8_t)block[2 + l];
                    if (!isfinite(w)) return TSO_E_NONFINITE;
                    sum += w * (xd ? xd[x0 + l] : (double)xf[x0 + l]);
                }
            } else {
                for (uint32_t l = 0; l < epb; ++l) {
                    const double w = tso_value(type, block, l);
                    if (!isfinite(w)) return TSO_E_NONFINITE;
                    sum += w * (xd ? xd[x0 + l] : (double)xf[x0 + l]);
                }
            }
        }
        if (!isfinite(sum)) return TSO_E_NONFINITE;
        output[row] = sum;
    }
    return TSO_OK;
}

int tso_gemv_f64(uint32_t type, const uint8_t* matrix, size_t nbytes, uint32_t columns, uint32_t rows,
                 const double* input, double* output) {
    return gemv_core(type, matrix, nbytes, columns, rows, input, NULL, output);
}
int tso_gemv_f32(uint32_t type, const uint8_t* matrix, size_t nbytes, uint32_t columns, uint32_t rows,
                 const float* input, double* output) {
    return gemv_core(type, matrix, nbytes, columns, rows, NULL, input, output);
}

/* operators.cpp:28-40 */
double tso_sigmoid(double v) {
    if (v >= 0) return 1 / (1 + exp(-v));
    const double p = exp(v);
    return p / (1 + p);
}
double tso_silu(double v) { return v * tso_sigmoid(v); }
double tso_softplus(double v) { return fmax(v, 0.0) + log1p(exp(-fabs(v))); }

/* routing.cpp:11-40. Selection by repeated scan instead of partial_sort: the k winners in
 * the total order (logit descending, id ascending) are the same set in the same order. */
int tso_route(const double* logits, size_t experts, size_t selected, uint32_t mode, int normalize,
              uint32_t* indices, double* weights) {
    if (!experts || experts > 4096 || !selected || selected > 64 || selected > experts || mode > 1) return TSO_E_SHAPE;
    for (size_t i = 0; i < experts; ++i) if (!isfinite(logits[i])) return TSO_E_NONFINITE;
    uint8_t taken[4096];
    memset(taken, 0, experts);
    for (size_t r = 0; r < selected; ++r) {
        size_t best = experts;
        for (size_t i = 0; i < experts; ++i) {
            if (taken[i]) continue;
            if (best == experts || logits[i] > logits[best]) best = i; /* strict > keeps the lower id on ties */
        }
        taken[best] = 1;
        indices[r] = (uint32_t)best;
    }
    const double maximum = logits[indices[0]];
    double act[64];
    for (size_t r = 0; r < selected; ++r) {
        const double l = logits[indices[r]];
        if (mode == 0) act[r] = exp(l - maximum);
        else if (normalize) act[r] = exp(-tso_softplus(-l) + tso_softplus(-maximum));
        else act[r] = tso_sigmoid(l);
    }
    double denominator = mode == 1 ? 1 : 0;
    if (normalize) {
        denominator = 0;
        for (size_t r = 0; r < selected; ++r) denominator += act[r];
    } else if (mode == 0) {
        for (size_t i = 0; i < experts; ++i) denominator += exp(logits[i] - maximum);
    }
    if (!isfinite(denominator) || denominator <= 0) return TSO_E_NONFINITE;
    for (size_t r = 0; r < selected; ++r) weights[r] = act[r] / denominator;
    return TSO_OK;
}

/* routing.cpp:42-61 */
/* operators.cpp:42-58 (grouped RMS), 60-89 (gated residual read), 91-96 (residual write) */
int tso_gated_residual(const double* streams, const double* gains, const double* down, const double* up, const double* inject,
                       size_t branches, size_t channels, size_t rank, double epsilon, double* input, double* write_scales,
                       double* normalized_out, double* scores_out, double* inject_out) {
    if (!branches || branches > 64 || !channels || channels > 65536 || !rank || rank > 4096 || !(epsilon > 0) || !isfinite(epsilon))
        return TSO_E_SHAPE;
    const size_t width = branches * channels;
    double* normalized = (double*)malloc(sizeof(double) * width);
    double* bottleneck = (double*)malloc(sizeof(double) * rank);
    if (!normalized || !bottleneck) { free(normalized); free(bottleneck); return TSO_E_SHAPE; }
    int rc = TSO_OK;
    for (size_t i = 0; i < width && !rc; ++i) if (!isfinite(streams[i]) || !isfinite(gains[i])) rc = TSO_E_NONFINITE;
    for (size_t g = 0; g < width && !rc; g += channels) {
        double squared = 0;
        for (size_t i = 0; i < channels; ++i) squared += streams[g + i] * streams[g + i];
        if (!isfinite(squared)) { rc = TSO_E_NONFINITE; break; }
        const double inverse = 1 / sqrt(squared / (double)channels + epsilon);
        for (size_t i = 0; i < channels; ++i) normalized[g + i] = streams[g + i] * inverse * gains[g + i];
    }
    for (size_t r = 0; r < rank && !rc; ++r) {
        double acc = 0;
        for (size_t i = 0; i < width; ++i) acc += down[r * width + i] * normalized[i];
        bottleneck[r] = tso_silu(acc / (double)branches);
    }
    for (size_t i = 0; i < channels && !rc; ++i) input[i] = 0;
    for (size_t b = 0; b < branches && !rc; ++b) {
        double scale = 0;
        for (size_t i = 0; i < width; ++i) scale += inject[b * width + i] * normalized[i];
        if (inject_out) inject_out[b] = scale;
        write_scales[b] = 2 * tso_sigmoid(scale / (double)branches);
    }
    for (size_t b = 0; b < branches && !rc; ++b)
        for (size_t c = 0; c < channels; ++c) {
            const size_t position = b * channels + c;
            double score = 0;
            for (size_t r = 0; r < rank; ++r) score += up[position * rank + r] * bottleneck[r];
            if (scores_out) scores_out[position] = score;
            input[c] += normalized[position] * tso_sigmoid(score) / (double)branches;
        }
    for (size_t i = 0; i < channels && !rc; ++i) if (!isfinite(input[i])) rc = TSO_E_NONFINITE;
    if (normalized_out && !rc) memcpy(normalized_out, normalized, sizeof(double) * width);
    free(normalized); free(bottleneck);
    return rc;
}

int tso_residual_write(const double* streams, const double* output, const double* scales, size_t branches, size_t channels, double* out) {
    if (!branches || !channels) return TSO_E_SHAPE;
    for (size_t b = 0; b < branches; ++b)
        for (size_t c = 0; c < channels; ++c) {
            const double v = streams[b * channels + c] + scales[b] * output[c];
            if (!isfinite(v)) return TSO_E_NONFINITE;
            out[b * channels + c] = v;
        }
    return TSO_OK;
}

int tso_mixture(const double* experts, const double* weights, size_t selected, const double* shared,
                size_t channels, double shared_logit, double* out) {
    if (!channels || channels > 65536 || !selected || selected > 64) return TSO_E_SHAPE;
    for (size_t r = 0; r < selected; ++r) if (!isfinite(weights[r]) || weights[r] < 0) return TSO_E_NONFINITE;
    if (!isfinite(shared_logit)) return TSO_E_NONFINITE;
    const double gate = tso_sigmoid(shared_logit);
    for (size_t c = 0; c < channels; ++c) {
        if (!isfinite(shared[c])) return TSO_E_NONFINITE;
        double v = gate * shared[c];
        for (size_t r = 0; r < selected; ++r) {
            const double y = experts[r * channels + c];
            if (!isfinite(y)) return TSO_E_NONFINITE;
            v += weights[r] * y;
        }
        if (!isfinite(v)) return TSO_E_NONFINITE;
        out[c] = v;
    }
    return TSO_OK;
}

/* sampling.cpp:473-515 */
static int topk_beats(float va, uint32_t ida, float vb, uint32_t idb) {
    const float ca = va == 0.0f ? 0.0f : va, cb = vb == 0.0f ? 0.0f : vb;   /* -0 and +0 compare as one value */
    return ca > cb || (ca == cb && ida < idb);
}

int tso_logit_topk_row(const float* logits, size_t vocabulary, tso_topk_row* out) {
    if (!vocabulary || vocabulary > ((size_t)1 << 20)) return TSO_E_SHAPE;
    memset(out, 0, sizeof *out);
    out->vocabulary = (uint32_t)vocabulary;
    out->first_nonfinite_col = out->first_subnormal_col = 0xffffffffu;
    for (int i = 0; i < TSO_TOPK_CAPACITY; ++i) out->logits[i] = -INFINITY;
    uint32_t count = 0;
    for (size_t i = 0; i < vocabulary; ++i) {
        const float raw = logits[i];
        uint32_t bits;
        memcpy(&bits, &raw, 4);
        const uint32_t exponent = bits & 0x7f800000u, mantissa = bits & 0x007fffffu, col = (uint32_t)i;
        if (exponent == 0x7f800000u) {
            if (out->first_nonfinite_col == 0xffffffffu) out->first_nonfinite_col = col;
            continue;
        }
        if (exponent == 0 && mantissa != 0 && out->first_subnormal_col == 0xffffffffu) out->first_subnormal_col = col;
        if (count == TSO_TOPK_CAPACITY && !topk_beats(raw, col, out->logits[count - 1], out->ids[count - 1])) continue;
        uint32_t pos = count < TSO_TOPK_CAPACITY ? count++ : TSO_TOPK_CAPACITY - 1;
        while (pos > 0 && topk_beats(raw, col, out->logits[pos - 1], out->ids[pos - 1])) {
            out->logits[pos] = out->logits[pos - 1];
            out->ids[pos] = out->ids[pos - 1];
            --pos;
        }
        out->logits[pos] = raw;
        out->ids[pos] = col;
    }
    out->count = count;
    return TSO_OK;
}

/* expert_lanes.cpp:75-130 (Q8_0 and Q4_K rows) */
static int lanes_geometry(uint32_t type, uint32_t columns, uint32_t* blocks, uint32_t* block_bytes, uint32_t* header, uint32_t* run) {
    if (type == 8u) { if (!columns || columns % 32 || columns > 65536) return TSO_E_SHAPE; *blocks = columns / 32; *block_bytes = 34; *header = 2; *run = 16; return TSO_OK; }
    if (type == 12u) { if (!columns || columns % 256 || columns > 65536) return TSO_E_SHAPE; *blocks = columns / 256; *block_bytes = 144; *header = 16; *run = 4; return TSO_OK; }
    return TSO_E_TYPE;
}
static uint64_t lanes_quant_offset(uint32_t type, uint32_t blocks, uint32_t meta, uint32_t block, uint32_t index) {
    if (type == 12u) {
        const uint32_t run = block / 4, left = blocks - run * 4, width = (left < 4 ? left : 4) * 4;
        const uint32_t pair = index / 32, lane = index % 32;
        return (uint64_t)meta + (uint64_t)run * 512 + lane * width + (block % 4) * 4 + pair;
    }
    const uint32_t run = block / 16, left = blocks - run * 16, width = left < 16 ? left : 16;
    return (uint64_t)meta + (uint64_t)run * 512 + index * width + block % 16;
}
static int lanes_move(uint32_t type, uint32_t columns, const uint8_t* in, uint8_t* out, size_t nbytes, int pack) {
    uint32_t blocks, bb, header, run;
    const int rc = lanes_geometry(type, columns, &blocks, &bb, &header, &run);
    if (rc) return rc;
    (void)run;
    const size_t row_bytes = (size_t)blocks * bb;
    const uint32_t meta = blocks * header;
    if (!nbytes || nbytes % row_bytes) return TSO_E_SHAPE;
    for (size_t row = 0; row < nbytes; row += row_bytes)
        for (uint32_t b = 0; b < blocks; ++b) {
            if (pack) memcpy(out + row + (size_t)b * header, in + row + (size_t)b * bb, header);
            else memcpy(out + row + (size_t)b * bb, in + row + (size_t)b * header, header);
            for (uint32_t i = 0; i < bb - header; ++i) {
                const uint64_t at = lanes_quant_offset(type, blocks, meta, b, i);
                if (pack) out[row + at] = in[row + (size_t)b * bb + header + i];
                else out[row + (size_t)b * bb + header + i] = in[row + at];
            }
        }
    return TSO_OK;
}
int tso_lanes_pack_rows(uint32_t type, uint32_t columns, const uint8_t* original, uint8_t* packed, size_t nbytes) {
    return lanes_move(type, columns, original, packed, nbytes, 1);
}
int tso_lanes_unpack_rows(uint32_t type, uint32_t columns, const uint8_t* packed, uint8_t* original, size_t nbytes) {
    return lanes_move(type, columns, packed, original, nbytes, 0);
}

/* ---- Pack v3 planar layout ---- */

/* planar_pack_v3.cpp:601-650 (Q4_K and Q8_0 rows of the table) */
int tso_make_expert_spec(uint32_t type, uint32_t columns, uint32_t rows, tso_planar_spec* s) {
    memset(s, 0, sizeof *s);
    if (rows < 4 || rows % 4) return TSO_E_SHAPE;
    s->source_type = type; s->columns = columns; s->rows = rows;
    if (type == 12) {
        if (columns < 256 || columns % 256) return TSO_E_SHAPE;
        s->blocks_per_row = columns / 256;
        const uint64_t total = (uint64_t)rows * s->blocks_per_row;
        s->source_row_bytes = (uint64_t)s->blocks_per_row * 144;
        s->planar_row_bytes = (uint64_t)s->blocks_per_row * 148;
        s->qs_offset = 0; s->sm_offset = total * 128; s->dm_offset = total * 144;
    } else if (type == 13) {   /* Q5_K: planes of nibbles, fifth bits, factor records, (d, dmin) pairs: 128 + 32 + 16 + 4 bytes per block */
        if (columns < 256 || columns % 256) return TSO_E_SHAPE;
        s->blocks_per_row = columns / 256;
        const uint64_t total = (uint64_t)rows * s->blocks_per_row;
        s->source_row_bytes = (uint64_t)s->blocks_per_row * 176;
        s->planar_row_bytes = (uint64_t)s->blocks_per_row * 180;
        s->qs_offset = 0; s->qh_offset = total * 128; s->sm_offset = total * 160; s->dm_offset = total * 176;
    } else if (type == 7) {    /* Q5_1: planes of nibbles, fifth-bit words, (d, m) pairs: 16 + 4 + 4 bytes per block */
        if (columns < 32 || columns % 32) return TSO_E_SHAPE;
        s->blocks_per_row = columns / 32;
        const uint64_t total = (uint64_t)rows * s->blocks_per_row;
        s->source_row_bytes = (uint64_t)s->blocks_per_row * 24;
        s->planar_row_bytes = s->source_row_bytes;
        s->qs_offset = 0; s->qh_offset = total * 16; s->dm_offset = total * 20;
    } else if (type == 8) {
        if (columns < 32 || columns % 32) return TSO_E_SHAPE;
        s->blocks_per_row = columns / 32;
        const uint64_t total = (uint64_t)rows * s->blocks_per_row;
        if (total % 8) return TSO_E_SHAPE;
        s->source_row_bytes = (uint64_t)s->blocks_per_row * 34;
        s->planar_row_bytes = s->source_row_bytes;
        s->qs_offset = 0; s->dm_offset = total * 32;
    } else return TSO_E_TYPE;
    s->source_expert_bytes = rows * s->source_row_bytes;
    s->planar_expert_bytes = rows * s->planar_row_bytes;
    if (s->planar_expert_bytes % 16) return TSO_E_SHAPE;
    return TSO_OK;
}

/* planar_pack_v3.cpp:652-661 */
void tso_pack_sm16(const uint8_t s12[12], uint8_t sm[16]) {
    for (int s = 0; s < 4; ++s) {
        sm[s] = s12[s] & 0x3f;
        sm[4 + s] = (uint8_t)((s12[8 + s] & 0x0f) | ((s12[s] >> 6) << 4));
        sm[8 + s] = s12[4 + s] & 0x3f;
        sm[12 + s] = (uint8_t)((s12[8 + s] >> 4) | ((s12[4 + s] >> 6) << 4));
    }
}

/* planar_pack_v3.cpp:663-674 */
int tso_unpack_sm16(const uint8_t sm[16], uint8_t s12[12]) {
    for (int i = 0; i < 16; ++i) if (sm[i] & 0xc0) return TSO_E_RANGE;
    for (int s = 0; s < 4; ++s) {
        s12[s] = (uint8_t)((sm[s] & 0x3f) | ((sm[4 + s] >> 4) << 6));
        s12[4 + s] = (uint8_t)((sm[8 + s] & 0x3f) | ((sm[12 + s] >> 4) << 6));
        s12[8 + s] = (uint8_t)((sm[4 + s] & 0x0f) | ((sm[12 + s] & 0x0f) << 4));
    }
    return TSO_OK;
}

/* planar_pack_v3.cpp:676-716 */
int tso_pack_expert_planar(const tso_planar_spec* s, const uint8_t* src, uint8_t* dst) {
    const uint64_t total = (uint64_t)s->rows * s->blocks_per_row;
    if (s->source_type == 12) {
        for (uint64_t b = 0; b < total; ++b) {
            const uint8_t* sb = src + b * 144;
            memcpy(dst + s->qs_offset + b * 128, sb + 16, 128);
            tso_pack_sm16(sb + 4, dst + s->sm_offset + b * 16);
            memcpy(dst + s->dm_offset + b * 4, sb, 4);
        }
    } else if (s->source_type == 13) {
        for (uint64_t b = 0; b < total; ++b) {
            const uint8_t* sb = src + b * 176;
            memcpy(dst + s->qs_offset + b * 128, sb + 48, 128);
            memcpy(dst + s->qh_offset + b * 32, sb + 16, 32);
            tso_pack_sm16(sb + 4, dst + s->sm_offset + b * 16);
            memcpy(dst + s->dm_offset + b * 4, sb, 4);
        }
    } else if (s->source_type == 7) {
        for (uint64_t b = 0; b < total; ++b) {
            const uint8_t* sb = src + b * 24;
            memcpy(dst + s->qs_offset + b * 16, sb + 8, 16);
            memcpy(dst + s->qh_offset + b * 4, sb + 4, 4);
            memcpy(dst + s->dm_offset + b * 4, sb, 4);
        }
    } else if (s->source_type == 8) {
        for (uint64_t b = 0; b < total; ++b) {
            const uint8_t* sb = src + b * 34;
            memcpy(dst + s->qs_offset + b * 32, sb + 2, 32);
            memcpy(dst + s->dm_offset + b * 2, sb, 2);
        }
    } else return TSO_E_TYPE;
    return TSO_OK;
}

/* planar_pack_v3.cpp:718-758 */
int tso_unpack_expert_planar(const tso_planar_spec* s, const uint8_t* src, uint8_t* dst) {
    const uint64_t total = (uint64_t)s->rows * s->blocks_per_row;
    if (s->source_type == 12) {
        for (uint64_t b = 0; b < total; ++b) {
            uint8_t* sb = dst + b * 144;
            memcpy(sb, src + s->dm_offset + b * 4, 4);
            const int rc = tso_unpack_sm16(src + s->sm_offset + b * 16, sb + 4);
            if (rc) return rc;
            memcpy(sb + 16, src + s->qs_offset + b * 128, 128);
        }
    } else if (s->source_type == 13) {
        for (uint64_t b = 0; b < total; ++b) {
            uint8_t* sb = dst + b * 176;
            memcpy(sb, src + s->dm_offset + b * 4, 4);
            const int rc = tso_unpack_sm16(src + s->sm_offset + b * 16, sb + 4);
            if (rc) return rc;
            memcpy(sb + 16, src + s->qh_offset + b * 32, 32);
            memcpy(sb + 48, src + s->qs_offset + b * 128, 128);
        }
    } else if (s->source_type == 7) {
        for (uint64_t b = 0; b < total; ++b) {
            uint8_t* sb = dst + b * 24;
            memcpy(sb, src + s->dm_offset + b * 4, 4);
            memcpy(sb + 4, src + s->qh_offset + b * 4, 4);
            memcpy(sb + 8, src + s->qs_offset + b * 16, 16);
        }
    } else if (s->source_type == 8) {
        for (uint64_t b = 0; b < total; ++b) {
            uint8_t* sb = dst + b * 34;
            memcpy(sb, src + s->dm_offset + b * 2, 2);
            memcpy(sb + 2, src + s->qs_offset + b * 32, 32);
        }
    } else return TSO_E_TYPE;
    return TSO_OK;
}

/* planar_pack_v3.cpp:760-830 */
int tso_dequantize_expert_planar(const tso_planar_spec* s, const uint8_t* base, float* out) {
    const uint64_t total = (uint64_t)s->rows * s->blocks_per_row;
    if (s->source_type == 12) {
        for (uint64_t b = 0; b < total; ++b) {
            const uint8_t* qs = base + s->qs_offset + b * 128;
            const uint8_t* sm = base + s->sm_offset + b * 16;
            const uint8_t* dm = base + s->dm_offset + b * 4;
            const double d = tso_binary16(rd16(dm)), dmin = tso_binary16(rd16(dm + 2));
            if (!isfinite(d) || !isfinite(dmin)) return TSO_E_NONFINITE;
            for (uint32_t g = 0; g < 8; ++g) {
                const double dl = d * sm[g], ml = dmin * sm[8 + g];
                const uint8_t* q = qs + (g >> 1) * 32;
                const uint32_t shift = (g & 1u) * 4u;
                for (uint32_t l = 0; l < 32; ++l) {
                    const float v = (float)(dl * ((q[l] >> shift) & 15u) - ml);
                    if (!isfinite(v)) return TSO_E_NONFINITE;
                    out[b * 256 + g * 32 + l] = v;
                }
            }
        }
    } else if (s->source_type == 13) {
        for (uint64_t b = 0; b < total; ++b) {
            const uint8_t* qs = base + s->qs_offset + b * 128;
            const uint8_t* qh = base + s->qh_offset + b * 32;
            const uint8_t* sm = base + s->sm_offset + b * 16;
            const uint8_t* dm = base + s->dm_offset + b * 4;
            const double d = tso_binary16(rd16(dm)), dmin = tso_binary16(rd16(dm + 2));
            if (!isfinite(d) || !isfinite(dmin)) return TSO_E_NONFINITE;
            for (uint32_t g = 0; g < 8; ++g) {
                const double dl = d * sm[g], ml = dmin * sm[8 + g];
                const uint8_t* q = qs + (g >> 1) * 32;
                const uint32_t shift = (g & 1u) * 4u;
                for (uint32_t l = 0; l < 32; ++l) {
                    const uint32_t code = ((q[l] >> shift) & 15u) | (((qh[l] >> g) & 1u) << 4);
                    const float v = (float)(dl * code - ml);
                    if (!isfinite(v)) return TSO_E_NONFINITE;
                    out[b * 256 + g * 32 + l] = v;
                }
            }
        }
    } else if (s->source_type == 7) {
        for (uint64_t b = 0; b < total; ++b) {
            const uint8_t* qs = base + s->qs_offset + b * 16;
            const uint32_t qh = rd32(base + s->qh_offset + b * 4);
            const uint8_t* dm = base + s->dm_offset + b * 4;
            const double d = tso_binary16(rd16(dm));
            const float m = tso_binary16(rd16(dm + 2));
            if (!isfinite(d) || !isfinite(m)) return TSO_E_NONFINITE;
            for (uint32_t i = 0; i < 32; ++i) {
                const uint32_t code = ((qs[i % 16] >> (4 * (i / 16))) & 15u) | (((qh >> i) & 1u) << 4);
                const float v = (float)(d * code + m);
                if (!isfinite(v)) return TSO_E_NONFINITE;
                out[b * 32 + i] = v;
            }
        }
    } else if (s->source_type == 8) {
        for (uint64_t b = 0; b < total; ++b) {
            const int8_t* qs = (const int8_t*)(base + s->qs_offset + b * 32);
            const double d = tso_binary16(rd16(base + s->dm_offset + b * 2));
            if (!isfinite(d)) return TSO_E_NONFINITE;
            for (uint32_t i = 0; i < 32; ++i) {
                const float v = (float)(d * qs[i]);
                if (!isfinite(v)) return TSO_E_NONFINITE;
                out[b * 32 + i] = v;
            }
        }
    } else return TSO_E_TYPE;
    return TSO_OK;
}

/* ---- permutation tables ---- */

/* grouped_mpp.metal:12-37: per expert, stable compaction over ascending token order. */
int tso_grouped_routes(const uint32_t* indices, uint32_t tokens, uint32_t experts, uint32_t selected,
                       uint32_t* token_map, uint32_t* counts) {
    int rc = TSO_OK;
    memset(counts, 0, (size_t)experts * 4);
    for (uint32_t t = 0; t < tokens; ++t) {
        for (uint32_t i = 0; i < selected; ++i) {
            const uint32_t id = indices[(size_t)t * selected + i];
            if (id >= experts) { rc = TSO_E_RANGE; continue; }
            for (uint32_t j = 0; j < i; ++j) if (indices[(size_t)t * selected + j] == id) rc = TSO_E_RANGE;
        }
    }
    if (rc) return rc;
    for (uint32_t t = 0; t < tokens; ++t)
        for (uint32_t i = 0; i < selected; ++i) {
            const uint32_t e = indices[(size_t)t * selected + i];
            token_map[(size_t)e * tokens + counts[e]++] = t * selected + i;
        }
    return TSO_OK;
}

/* grouped_mpp.metal:41-66 */
int tso_grouped_tasks(const uint32_t* counts, uint32_t tokens, uint32_t experts, uint32_t selected,
                      uint32_t tile, uint32_t* tasks) {
    if (!tile) return TSO_E_SHAPE;
    const uint32_t bound = tokens * selected / tile + experts;
    uint32_t total = 0, routes = 0;
    for (uint32_t i = 0; i < bound; ++i) { tasks[2 + 2 * i] = UINT32_MAX; tasks[3 + 2 * i] = UINT32_MAX; }
    int rc = TSO_OK;
    for (uint32_t e = 0; e < experts; ++e) {
        if (counts[e] > tokens) rc = TSO_E_RANGE;
        const uint32_t c = counts[e] < tokens ? counts[e] : tokens;
        const uint32_t n = (c + tile - 1) / tile;
        for (uint32_t i = 0; i < n; ++i) if (total + i < bound) { tasks[2 + 2 * (total + i)] = e; tasks[3 + 2 * (total + i)] = i * tile; }
        total += n; routes += counts[e];
    }
    tasks[0] = total < bound ? total : bound;
    tasks[1] = routes;
    if (total > bound || routes != tokens * selected) rc = TSO_E_RANGE;
    return rc;
}

/* ---- whole layer (ffn_check.cpp:104-139), threaded over token rows ---- */

typedef struct {
    const tso_layer* L; const float* x; const float* logits; uint32_t t0, t1;
    double* out; const tso_layer_stages* st; int rc;
} layer_job;

static size_t tensor_bytes(uint32_t type, uint64_t elements) {
    uint32_t epb, bpb;
    if (tso_block_geometry(type, &epb, &bpb)) return 0;
    return (size_t)(elements / epb) * bpb;
}

static void* layer_worker(void* arg) {
    layer_job* j = (layer_job*)arg;
    const tso_layer* L = j->L;
    const uint32_t C = L->channels, H = L->hidden, E = L->experts, K = L->selected;
    const size_t gu_bytes = tensor_bytes(L->expert_type, (uint64_t)C * H);
    const uint32_t down_type = L->down_type ? L->down_type : L->expert_type;
    const size_t dn_bytes = tensor_bytes(down_type, (uint64_t)C * H);
    const size_t sgu_bytes = tensor_bytes(L->shared_type, (uint64_t)C * H);
    double* xd = (double*)malloc(sizeof(double) * C);
    double* lg = (double*)malloc(sizeof(double) * E);
    double* g = (double*)malloc(sizeof(double) * H);
    double* u = (double*)malloc(sizeof(double) * H);
    double* routed = (double*)malloc(sizeof(double) * (size_t)K * C);
    double* sh = (double*)malloc(sizeof(double) * C);
    uint32_t ids[64]; double w[64];
    j->rc = TSO_OK;
    for (uint32_t t = j->t0; t < j->t1 && !j->rc; ++t) {
        int rc = TSO_OK;
        for (uint32_t c = 0; c < C; ++c) xd[c] = j->x[(size_t)t * C + c];
        if (j->logits) for (uint32_t e = 0; e < E; ++e) lg[e] = j->logits[(size_t)t * E + e];
        else rc = tso_gemv_f64(0, (const uint8_t*)L->router, (size_t)E * C * 4, C, E, xd, lg);
        if (!rc) rc = tso_route(lg, E, K, L->mode, L->normalize_selected, ids, w);
        for (uint32_t r = 0; r < K && !rc; ++r) {
            const uint32_t e = ids[r];
            rc = tso_gemv_f64(L->expert_type, L->gate + (size_t)e * gu_bytes, gu_bytes, C, H, xd, g);
            if (!rc) rc = tso_gemv_f64(L->expert_type, L->up + (size_t)e * gu_bytes, gu_bytes, C, H, xd, u);
            if (rc) break;
            for (uint32_t i = 0; i < H; ++i) g[i] = tso_silu(g[i]) * u[i];
            if (j->st && j->st->activated) memcpy(j->st->activated + ((size_t)t * K + r) * H, g, sizeof(double) * H);
            rc = tso_gemv_f64(down_type, L->down + (size_t)e * dn_bytes, dn_bytes, H, C, g, routed + (size_t)r * C);
        }
        if (!rc) rc = tso_gemv_f64(L->shared_type, L->shared_gate, sgu_bytes, C, H, xd, g);
        if (!rc) rc = tso_gemv_f64(L->shared_type, L->shared_up, sgu_bytes, C, H, xd, u);
        if (!rc) {
            for (uint32_t i = 0; i < H; ++i) g[i] = tso_silu(g[i]) * u[i];
            rc = tso_gemv_f64(L->shared_type, L->shared_down, sgu_bytes, H, C, g, sh);
        }
        double slogit = 0;
        if (!rc && L->shared_router) rc = tso_gemv_f64(0, (const uint8_t*)L->shared_router, (size_t)C * 4, C, 1, xd, &slogit);
        if (!rc) rc = tso_mixture(routed, w, K, sh, C, slogit, j->out + (size_t)t * C);
        if (!rc && j->st) {
            const tso_layer_stages* s = j->st;
            if (s->indices) memcpy(s->indices + (size_t)t * K, ids, 4 * K);
            if (s->weights) memcpy(s->weights + (size_t)t * K, w, sizeof(double) * K);
            if (s->routed) memcpy(s->routed + (size_t)t * K * C, routed, sizeof(double) * (size_t)K * C);
            if (s->shared_act) memcpy(s->shared_act + (size_t)t * H, g, sizeof(double) * H);
            if (s->shared_out) memcpy(s->shared_out + (size_t)t * C, sh, sizeof(double) * C);
            if (s->shared_logit) s->shared_logit[t] = slogit;
        }
        j->rc = rc;
    }
    free(xd); free(lg); free(g); free(u); free(routed); free(sh);
    return NULL;
}

int tso_moe_layer(const tso_layer* L, const float* x, const float* logits, uint32_t tokens,
                  double* out, const tso_layer_stages* stages, uint32_t threads) {
    if (!L->channels || !L->hidden || !L->experts || !L->selected || L->selected > 64 || L->selected > L->experts ||
        L->experts > 4096 || !tokens || (!logits && !L->router)) return TSO_E_SHAPE;
    if (!threads) threads = 1;
    if (threads > tokens) threads = tokens;
    if (threads > 256) threads = 256;
    layer_job jobs[256];
    pthread_t tid[256];
    for (uint32_t i = 0; i < threads; ++i) {
        jobs[i] = (layer_job){L, x, logits, (uint32_t)((uint64_t)tokens * i / threads),
                              (uint32_t)((uint64_t)tokens * (i + 1) / threads), out, stages, 0};
        if (i + 1 < threads) pthread_create(&tid[i], NULL, layer_worker, &jobs[i]);
    }
    layer_worker(&jobs[threads - 1]);
    int rc = jobs[threads - 1].rc;
    for (uint32_t i = 0; i + 1 < threads; ++i) { pthread_join(tid[i], NULL); if (jobs[i].rc) rc = jobs[i].rc; }
    return rc;
}
