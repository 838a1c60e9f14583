// Test infrastructure, not product code.
//
// Re-exports the reference's speculative-decoding host classes (SuffixIndex,
// src/spec/suffix_index.h:16-114; SpecController, src/spec/spec_controller.h:16-107;
// both header-only, included from where the reference checkout lies) through a
// C ABI, so that the CPU tests can drive them and the library's versions with the
// same sequences of calls. Nothing from the reference is copied here.
#include "spec/suffix_index.h"
#include "spec/spec_controller.h"

using fastllm::SpecController;
using fastllm::SuffixIndex;

extern "C" {

void *flref_suffix_create(uint32_t chain_cap, uint32_t min_match) { return new SuffixIndex(chain_cap, min_match); }
void flref_suffix_destroy(void *h) { delete (SuffixIndex *)h; }
void flref_suffix_reset(void *h) { ((SuffixIndex *)h)->reset(); }
void flref_suffix_push(void *h, int32_t t) { ((SuffixIndex *)h)->push(t); }
uint64_t flref_suffix_size(void *h) { return ((SuffixIndex *)h)->size(); }
int flref_suffix_draft(void *h, int n_max, int32_t *out, int32_t *diag) {
    SuffixIndex::Diag dg;
    const int n = ((const SuffixIndex *)h)->draft(n_max, out, &dg);
    if (diag) { diag[0] = dg.gram_seen; diag[1] = dg.cands; diag[2] = dg.best_len; diag[3] = dg.walked; }
    return n;
}

void *flref_spec_create(int n_max, double alpha0, double alpha_decay, double lat_decay, int probe_iv, int probe_n,
                        double seed_slope) {
    SpecController::Cfg c;
    c.n_max = n_max; c.alpha0 = alpha0; c.alpha_decay = alpha_decay; c.lat_decay = lat_decay;
    c.probe_iv = probe_iv; c.probe_n = probe_n; c.seed_slope = seed_slope;
    return new SpecController(c);
}
void flref_spec_destroy(void *h) { delete (SpecController *)h; }
int flref_spec_choose(void *h) { return ((SpecController *)h)->choose(); }
void flref_spec_observe(void *h, int nd, int na, double ms) { ((SpecController *)h)->observe(nd, na, ms); }
double flref_spec_alpha(void *h) { return ((SpecController *)h)->alpha(); }
double flref_spec_lat_est(void *h, int n) { return ((SpecController *)h)->lat_est(n); }
double flref_spec_expected_emitted(void *h, int n) { return ((SpecController *)h)->expected_emitted(n); }

} // extern "C"
