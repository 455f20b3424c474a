/*
 * oracle/ref_drafter_harness.c — TEST INFRASTRUCTURE, never linked into the product.
 *
 * Reaches the reference's n-gram drafter, a file-local function of src/engine/session.c
 * (propose_drafts_ngram, session.c:437-513), by textually including that translation unit
 * (found through -I at build time; nothing is copied). Built with hidden visibility and
 * section garbage collection, so that everything of the engine that the drafter does not
 * call is dropped at link time and the library loads without the engine.
 */
#include "src/engine/session.c" /* the reference TU itself */

__attribute__((visibility("default"))) size_t ref_propose_drafts_ngram(const geist_token_t *history, size_t history_n, geist_token_t seed, size_t k_max, size_t max_suffix,
                                                                       geist_token_t *out, size_t *out_match_L) {
    return propose_drafts_ngram(history, history_n, seed, k_max, max_suffix, out, out_match_L);
}
