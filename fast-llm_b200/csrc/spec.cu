// Speculative decoding around the decoder's batch pass: the draft source, the
// draft-length controller and the generation loop. Host code only.
//
//   draft source  longest-suffix match over the token stream so far (class SuffixIndex of the reference,
//                 src/spec/suffix_index.h:16-114): same definition, same results, including what a
//                 bounded walk over the occurrences of the tail's 3-gram examines
//   controller    class SpecController (src/spec/spec_controller.h:16-107): n = argmax of expected
//                 emitted tokens / measured pass latency, forced probes after draftless rounds
//   loop          the speculative branch of the reference's decode tool (tools/decode_main.cpp:329-400),
//                 without its margin gate: every position of this decoder's batch pass is exact
#include "capi_internal.h"

#include <chrono>
#include <cstring>
#include <unordered_map>
#include <vector>

using namespace flb;

namespace {

constexpr size_t kGram = 3;   // tokens per indexed gram

// Occurrence lists are threaded through `older`: older[e] is the previous position at which a gram with the same
// key ended. Keys are a 64-bit mix of the gram, so an entry is compared token by token before it counts.
struct GramKeyMix {
    static uint64_t of(const int32_t *g) {
        uint64_t x = 0;
        for (size_t i = 0; i < kGram; ++i) {   // multiply / xor-shift rounds over the three tokens
            x = (x + (uint32_t)g[i] + 1u) * 0xD6E8FEB86659FD93ull;
            x ^= x >> 29;
        }
        return x;
    }
};

} // namespace

struct fl_b200_suffix {
    uint32_t walk_limit = 64, min_match = 3;
    std::vector<int32_t> stream;
    std::vector<int64_t> older;                       // per end position
    std::unordered_map<uint64_t, int64_t> newest;     // key -> most recent end position
};

struct fl_b200_spec {
    static constexpr int kBuckets = 16;               // draft lengths 0..15
    fl_b200_spec_cfg cfg;
    double alpha;
    double lat_ms[kBuckets];                          // < 0: nothing measured yet
    int draftless_rounds = 0;
    static int bucket(int n) { return n < 0 ? 0 : n >= kBuckets ? kBuckets - 1 : n; }
};

extern "C" {

int fl_b200_suffix_create(uint32_t chain_cap, uint32_t min_match, fl_b200_suffix **out) {
    if (!out) return set_err(FL_B200_ERR_ARG, "suffix_create: null");
    fl_b200_suffix *s = new fl_b200_suffix();
    s->walk_limit = chain_cap;
    s->min_match = min_match;
    *out = s;
    return FL_B200_OK;
}

void fl_b200_suffix_destroy(fl_b200_suffix *s) { delete s; }

void fl_b200_suffix_reset(fl_b200_suffix *s) {
    if (!s) return;
    s->stream.clear();
    s->older.clear();
    s->newest.clear();
}

void fl_b200_suffix_push(fl_b200_suffix *s, int32_t tok) {
    if (!s) return;
    s->stream.push_back(tok);
    s->older.push_back(-1);
    const size_t n = s->stream.size();
    if (n < kGram) return;
    const uint64_t key = GramKeyMix::of(&s->stream[n - kGram]);
    auto ins = s->newest.emplace(key, (int64_t)(n - 1));
    if (!ins.second) {
        s->older[n - 1] = ins.first->second;
        ins.first->second = (int64_t)(n - 1);
    }
}

uint64_t fl_b200_suffix_size(const fl_b200_suffix *s) { return s ? s->stream.size() : 0; }

int fl_b200_suffix_draft(const fl_b200_suffix *s, int32_t n_max, int32_t *out, int32_t *diag) {
    int32_t dg[4] = {0, 0, 0, 0};   // tail gram indexed, candidates compared, longest match, entries walked
    auto done = [&](int r) { if (diag) memcpy(diag, dg, sizeof dg); return r; };
    if (!s || !out) return done(0);
    const std::vector<int32_t> &t = s->stream;
    const size_t n = t.size();
    if (n < kGram || n_max <= 0) return done(0);
    const auto head = s->newest.find(GramKeyMix::of(&t[n - kGram]));
    if (head == s->newest.end()) return done(0);
    dg[0] = 1;
    const int64_t tail = (int64_t)n - 1;
    int64_t match_end = -1;
    size_t match_len = 0;
    uint32_t walked = 0;
    // newest first, so among equally long matches the first one found (the most recent) stays; the tail's
    // own entry (and an entry of a colliding key, should one ever occur) uses up walk budget like any other
    for (int64_t e = head->second; e >= 0 && walked < s->walk_limit; e = s->older[(size_t)e], ++walked) {
        if (e == tail) continue;
        if (memcmp(&t[(size_t)e + 1 - kGram], &t[n - kGram], kGram * sizeof(int32_t)) != 0) continue;
        size_t len = kGram;   // grow the match towards the start of the stream
        while (len <= (size_t)e && len < n - 1 && t[(size_t)e - len] == t[(size_t)tail - len]) ++len;
        ++dg[1];
        if (len > match_len) { match_len = len; match_end = e; }
    }
    dg[2] = (int32_t)match_len;
    dg[3] = (int32_t)walked;
    if (match_end < 0 || match_len < s->min_match) return done(0);
    int32_t cnt = 0;
    for (size_t p = (size_t)match_end + 1; p < n && cnt < n_max; ++p) out[cnt++] = t[p];
    return done(cnt);
}

void fl_b200_spec_cfg_default(fl_b200_spec_cfg *c) {
    if (!c) return;
    c->n_max = 7; c->alpha0 = 0.75; c->alpha_decay = 0.90; c->lat_decay = 0.80; c->probe_iv = 16; c->probe_n = 2;
    c->seed_slope = 0.15;
}

int fl_b200_spec_create(const fl_b200_spec_cfg *cfg, fl_b200_spec **out) {
    if (!out) return set_err(FL_B200_ERR_ARG, "spec_create: null");
    fl_b200_spec *s = new fl_b200_spec();
    if (cfg) s->cfg = *cfg; else fl_b200_spec_cfg_default(&s->cfg);
    s->alpha = s->cfg.alpha0;
    for (double &l : s->lat_ms) l = -1.0;
    *out = s;
    return FL_B200_OK;
}

void fl_b200_spec_destroy(fl_b200_spec *s) { delete s; }

double fl_b200_spec_alpha(const fl_b200_spec *s) { return s ? s->alpha : 0.0; }

// 1 + alpha + ... + alpha^n: the accepted geometric prefix plus the correction token.
double fl_b200_spec_expected_emitted(const fl_b200_spec *s, int32_t n) {
    if (!s) return 0.0;
    double sum = 0.0, term = 1.0;
    for (int i = 0; i <= n; ++i) { sum += term; term *= s->alpha; }
    return sum;
}

// Latency of a pass with n drafts: the bucket's running mean, else the nearest measured bucket scaled by
// (1 + seed_slope * distance) (lower buckets first), else 1.
double fl_b200_spec_lat_est(const fl_b200_spec *s, int32_t n) {
    if (!s) return 1.0;
    const int b = fl_b200_spec::bucket(n), last = fl_b200_spec::kBuckets - 1;
    if (s->lat_ms[b] >= 0.0) return s->lat_ms[b];
    for (int dist = 1; dist <= last; ++dist) {
        const double grow = 1.0 + s->cfg.seed_slope * dist;
        if (b - dist >= 0 && s->lat_ms[b - dist] >= 0.0) return s->lat_ms[b - dist] * grow;
        if (b + dist <= last && s->lat_ms[b + dist] >= 0.0) return s->lat_ms[b + dist] / grow;
    }
    return 1.0;
}

int32_t fl_b200_spec_choose(fl_b200_spec *s) {
    if (!s) return 0;
    if (s->lat_ms[0] < 0.0) return s->cfg.n_max;   // nothing known about a draftless pass yet: try a full draft
    int pick = 0;
    double rate = 1.0 / fl_b200_spec_lat_est(s, 0);
    for (int n = 1; n <= s->cfg.n_max; ++n) {
        const double r = fl_b200_spec_expected_emitted(s, n) / fl_b200_spec_lat_est(s, n);
        if (r > rate) { rate = r; pick = n; }
    }
    if (pick != 0) {
        s->draftless_rounds = 0;
        return pick;
    }
    if (++s->draftless_rounds >= s->cfg.probe_iv) {   // keep the acceptance estimate from going stale
        s->draftless_rounds = 0;
        return s->cfg.probe_n;
    }
    return 0;
}

void fl_b200_spec_observe(fl_b200_spec *s, int32_t n_drafted, int32_t n_accepted, double pass_ms) {
    if (!s) return;
    double &lat = s->lat_ms[fl_b200_spec::bucket(n_drafted)];
    lat = lat < 0.0 ? pass_ms : s->cfg.lat_decay * lat + (1.0 - s->cfg.lat_decay) * pass_ms;
    if (n_drafted <= 0) return;
    const double frac = (double)n_accepted / (double)n_drafted;
    s->alpha = s->cfg.alpha_decay * s->alpha + (1.0 - s->cfg.alpha_decay) * frac;
    if (s->alpha < 0.02) s->alpha = 0.02;
    if (s->alpha > 0.98) s->alpha = 0.98;
}

int fl_b200_decoder_generate_spec(fl_b200_decoder *dec, int32_t first_token, uint32_t n_gen, int32_t spec_max,
                                  int32_t spec_fixed, fl_b200_suffix *idx, fl_b200_spec *ctrl, int32_t *out_tokens,
                                  fl_b200_spec_stats *stats) {
    if (!dec || !idx || !out_tokens) return set_err(FL_B200_ERR_ARG, "generate_spec: null");
    if (spec_fixed < 0 && !ctrl) return set_err(FL_B200_ERR_ARG, "generate_spec: a controller is needed unless the draft length is fixed");
    if (spec_max < 0 || spec_max > FL_B200_MAX_BATCH - 1)
        return set_err(FL_B200_ERR_ARG, "generate_spec: spec_max %d outside 0..%d", spec_max, FL_B200_MAX_BATCH - 1);
    fl_b200_spec_stats st;
    memset(&st, 0, sizeof st);
    int32_t toks[FL_B200_MAX_BATCH], outs[FL_B200_MAX_BATCH], draft[FL_B200_MAX_BATCH];
    int32_t next = first_token;   // emitted at the top of a round, fed to the model in that round's pass
    uint32_t n_out = 0;
    int rc = FL_B200_OK;
    while (n_out < n_gen) {
        out_tokens[n_out++] = next;
        if (n_out >= n_gen) break;
        fl_b200_suffix_push(idx, next);
        int32_t want = spec_fixed >= 0 ? spec_fixed : fl_b200_spec_choose(ctrl);
        if (want > spec_max) want = spec_max;
        const int32_t nd = want > 0 ? fl_b200_suffix_draft(idx, want, draft, nullptr) : 0;
        toks[0] = next;
        for (int32_t k = 0; k < nd; ++k) toks[k + 1] = draft[k];
        int32_t base = 0;
        if ((rc = fl_b200_decoder_n_past(dec, &base))) break;
        const auto t0 = std::chrono::steady_clock::now();
        if ((rc = fl_b200_decoder_step_batch(dec, toks, (uint32_t)nd + 1, outs, nullptr))) break;
        const double pass_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        int32_t acc = 0;
        while (acc < nd && outs[acc] == draft[acc]) ++acc;
        for (int32_t k = 0; k < acc && n_out < n_gen; ++k) {
            out_tokens[n_out++] = draft[k];
            fl_b200_suffix_push(idx, draft[k]);
        }
        next = outs[acc];   // the model's own token after the accepted prefix
        if ((rc = fl_b200_decoder_set_n_past(dec, base + acc + 1))) break;   // rows of rejected drafts are dropped
        if (spec_fixed < 0) fl_b200_spec_observe(ctrl, nd, acc, pass_ms);
        ++st.passes;
        st.drafted += (uint32_t)nd;
        st.accepted += (uint32_t)acc;
        ++st.n_hist[nd > 16 ? 16 : nd];
        st.pass_ms += pass_ms;
    }
    st.emitted = n_out;
    if (stats) *stats = st;
    return rc;
}

} // extern "C"
