// Host-side ingestion of packed SEED4P4 weights (include/nslm_pack.h): bank files -> streams, streams -> slice tables.
#include "common.cuh"
#include "../../include/nslm_pack.h"

#include <cstring>

using namespace nsl;

static_assert(sizeof(NslBlkHeader) == 56, "bank header layout");

extern "C" {

size_t nsl_blk4_bytes(int n_experts, int rows, int cols) {
    const size_t e = (size_t) n_experts, nb = (size_t) rows * (size_t) cols / 8;
    return sizeof(NslBlkHeader) + 12 * e + 5 * nb * e;
}

int nsl_blk4_split(const void* blk, size_t len, int n_experts, int rows, int cols, uint16_t* seeds, uint16_t* coefs,
                   int32_t* exp_bias, uint8_t* codes) {
    if (!blk || n_experts < 1 || rows < 1 || cols < 8 || cols % 8) return -1;
    const size_t e = (size_t) n_experts, nb = (size_t) rows * (size_t) cols / 8;
    NslBlkHeader h;
    if (len != nsl_blk4_bytes(n_experts, rows, cols)) return -1;
    memcpy(&h, blk, sizeof h);
    if (memcmp(h.magic, "NSLMBLK4", 8) || h.rows != (uint32_t) rows || h.cols != (uint32_t) cols || h.n_experts != (uint32_t) n_experts)
        return -1;
    const uint8_t* base = (const uint8_t*) blk + sizeof h;
    const uint8_t* sp = base + 12 * e, *cp = sp + 2 * nb * e, *ec = cp + 2 * nb * e;
    if (exp_bias) memcpy(exp_bias, base, 4 * e);
    if (seeds) memcpy(seeds, sp, 2 * nb * e);
    if (coefs) memcpy(coefs, cp, 2 * nb * e);
    if (codes)
        for (size_t k = 0; k < nb * e; k += 2)      // two codes per byte, block 2j in the low nibble
            codes[k / 2] = (uint8_t) ((ec[k] & 15) | ((k + 1 < nb * e ? ec[k + 1] & 15 : 0) << 4));
    return 0;
}

int nsl_blk4_join(void* blk, size_t len, int n_experts, int rows, int cols, const uint16_t* seeds, const uint16_t* coefs,
                  const int32_t* exp_bias, const uint8_t* codes) {
    if (!blk || !seeds || !coefs || !exp_bias || !codes || n_experts < 1 || rows < 1 || cols < 8 || cols % 8 ||
        len != nsl_blk4_bytes(n_experts, rows, cols))
        return -1;
    const size_t e = (size_t) n_experts, nb = (size_t) rows * (size_t) cols / 8;
    memset(blk, 0, len);
    NslBlkHeader h;
    memset(&h, 0, sizeof h);
    memcpy(h.magic, "NSLMBLK4", 8);
    h.rows = (uint32_t) rows; h.cols = (uint32_t) cols; h.n_experts = (uint32_t) n_experts;
    memcpy(blk, &h, sizeof h);
    uint8_t* base = (uint8_t*) blk + sizeof h;
    uint8_t* sp = base + 12 * e, *cp = sp + 2 * nb * e, *ec = cp + 2 * nb * e;
    memcpy(base, exp_bias, 4 * e);
    memcpy(sp, seeds, 2 * nb * e);
    memcpy(cp, coefs, 2 * nb * e);
    for (size_t k = 0; k < nb * e; ++k) ec[k] = (uint8_t) ((codes[k / 2] >> ((k & 1) * 4)) & 15);
    return 0;
}

int nsl_wslice_table(const void* seeds, const void* coefs, const void* codes, const int32_t* exp_bias, int slices, int rows,
                     int cols, WSlice* table) {
    if (!seeds || !coefs || !codes || !exp_bias || !table || slices < 1 || rows < 1 || cols < 8 ||
        ((size_t) rows * (size_t) cols) % 16) {
        set_error("nsl_wslice_table: %d slices of %d x %d (rows * cols must be a multiple of 16) or a missing stream", slices, rows, cols);
        return -1;
    }
    const size_t nb = (size_t) rows * (size_t) cols / 8;
    for (int i = 0; i < slices; ++i) {
        memset(&table[i], 0, sizeof(WSlice));
        table[i].p[0] = (const uint16_t*) seeds + (size_t) i * nb;
        table[i].p[1] = (const uint16_t*) coefs + (size_t) i * nb;
        table[i].p[3] = (const uint8_t*) codes + (size_t) i * (nb / 2);
        table[i].eb = exp_bias[i];
    }
    return 0;
}

}   // extern "C"
