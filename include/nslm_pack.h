/* nslm_pack.h - feeding packed SEED4P4 weights to the kernels: the expert bank files of the reference's compressor and
 * the slice tables its engine builds at load time.  Host code only (no launches).
 *
 * Stream layout of a SEED4P4 tensor (nslm/model_st.h:13-16): seeds u16 [slices][rows][cols/8], coefficient words u16
 * [slices][rows][cols/8], exponent biases i32 [slices], exponent codes u8 [slices][rows][cols/16] (two 4-bit codes per
 * byte, the even block in the low nibble). */
#pragma once
#include "nslm_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Header of a .blk4 bank (nslm/moe.h:10-17; 56 bytes, field order is the format).  After it: 12 bytes per expert, of
 * which the first 4 n_experts are the experts' i32 exponent biases (the other 8 n_experts bytes are not read here),
 * then all experts' seeds (u16 per block), coefficient words (u16 per block) and exponent codes (ONE BYTE per
 * block), experts in order. */
typedef struct {
    char magic[8];               /* "NSLMBLK4" */
    uint32_t rows, cols, n_experts;
    uint32_t n_seeds, n_exp, refit;
    int32_t exp_delta[3];
    float n0;
    double seconds;
} NslBlkHeader;

/* nslm/lib_moe.c:92-107 (nslm_blk_stream, p = 4), all four streams at once: splits a .blk4 image of n_experts experts
 * of rows x cols into seeds / coefs [n_experts][rows*cols/8], exp_bias [n_experts] and codes [n_experts*rows*cols/16]
 * (repacked two per byte, block 2j in the low nibble).  Any output may be NULL.  0, or -1 when the image's magic, shape
 * or length do not match. */
int nsl_blk4_split(const void* blk, size_t len, int n_experts, int rows, int cols, uint16_t* seeds, uint16_t* coefs,
                   int32_t* exp_bias, uint8_t* codes);
/* The inverse, for tests and tools: builds a .blk4 image (len = nsl_blk4_bytes) from the four streams. */
size_t nsl_blk4_bytes(int n_experts, int rows, int cols);
int nsl_blk4_join(void* blk, size_t len, int n_experts, int rows, int cols, const uint16_t* seeds, const uint16_t* coefs,
                  const int32_t* exp_bias, const uint8_t* codes);
/* engine/qwen4_cuda.c:197-216 (load_w): the slice table of a tensor whose streams lie at seeds / coefs / codes (device
 * or mapped host addresses; slice i's streams start i * rows*cols/8 elements in, codes i * rows*cols/16 bytes in) with
 * exponent biases exp_bias (host memory): table[i] = {p = {seeds_i, coefs_i, NULL, codes_i}, eb = exp_bias[i]}.
 * rows * cols must be a multiple of 16.  0 or -1. */
int nsl_wslice_table(const void* seeds, const void* coefs, const void* codes, const int32_t* exp_bias, int slices, int rows,
                     int cols, WSlice* table);

#ifdef __cplusplus
}
#endif
