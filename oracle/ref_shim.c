/* Thin flat-argument entry points over the reference's own C sources, compiled where they lie (never copied) into
 * oracle/_ref/libnslm_ref.so by oracle/Makefile.  TEST INFRASTRUCTURE ONLY: used to validate the oracle restatement
 * and to generate the golden fixtures under tests/golden/.  The reference headers are found with -I at build time. */
#include <stdint.h>
#include <string.h>

#include "lfsr.h"
#include "qwen4_cfg.h"
#include "qwen4_ops.h"
#include "rows.h"
#include "search4.h"

void ref_states(uint16_t s, int n, uint16_t* out) { lfsr_states(s, n, out); }
uint32_t ref_stream32(uint16_t s) { return lfsr_stream32(s); }
void ref_decode_block(uint16_t seed, uint16_t coef, int e, uint16_t* out) { nslm4_decode_block(seed, coef, e, out); }

/* One f32 row of a single-slice SEED4P4 matrix through the reference's weight reader (ns_row_f32). */
void ref_row_f32(const uint16_t* seeds, const uint16_t* coefs, const uint8_t* codes, int32_t eb, int rows, int K, int row,
                 float* out) {
    static NsRows tables;
    static int ready;
    if (!ready) { ns_rows_init(&tables); ready = 1; }
    NsTensor t;
    memset(&t, 0, sizeof t);
    t.enc = NS_SEED4P4;
    t.slices = 1;
    t.rows = rows;
    t.cols = K;
    t.s[0].p = (const uint8_t*) seeds;
    t.s[1].p = (const uint8_t*) coefs;
    t.s[2].p = (const uint8_t*) &eb;
    t.s[3].p = codes;
    ns_row_f32(&tables, &t, 0, row, 0, out);
}

/* P = 3 (SEED4): the spec's block decode and a row through the reference's weight reader. */
void ref_decode3_block(uint16_t seed, uint16_t nib, int bias, uint16_t* out) { nslm_decode_block(seed, nib, bias, out); }
void ref_row3_f32(const uint16_t* seeds, const uint16_t* nibs, int32_t eb, int rows, int K, int row, float* out) {
    static NsRows tables;
    static int ready;
    if (!ready) { ns_rows_init(&tables); ready = 1; }
    NsTensor t;
    memset(&t, 0, sizeof t);
    t.enc = NS_SEED4;
    t.slices = 1;
    t.rows = rows;
    t.cols = K;
    t.s[0].p = (const uint8_t*) seeds;
    t.s[1].p = (const uint8_t*) nibs;
    t.s[2].p = (const uint8_t*) &eb;
    ns_row_f32(&tables, &t, 0, row, 0, out);
}

void ref_route(int E, int k, const float* logits, int32_t* ind, float* wt) {
    Qwen4Cfg c;
    memset(&c, 0, sizeof c);
    c.n_exp = E;
    c.top_k = k;
    qwen4_route(&c, logits, ind, wt);
}
