// Test shim: the C++ target adapter (include/pyre_b200_target.hpp) behind a few C entry points, so that the Python tests can drive
// it on handles they made through the ctypes mirror and compare it with that mirror.
#include <cstring>

#include "pyre_b200_target.hpp"

using pyre_b200::QnTarget;

extern "C" {
void* shim_make(void* ctx, void* model, void* state) {
    try { return new QnTarget(static_cast<pb_ctx*>(ctx), static_cast<pb_model*>(model), static_cast<pb_state*>(state)); } catch (...) { return nullptr; }
}
void shim_free(void* t) { delete static_cast<QnTarget*>(t); }
int shim_caps(void* t, int* can_verify, long long* max_window) {
    QnTarget* q = static_cast<QnTarget*>(t);
    *can_verify = q->can_verify() ? 1 : 0;
    *max_window = static_cast<long long>(q->max_window());
    return 0;
}
int shim_step(void* t, unsigned tok, float* logits, int n) {
    try { auto lg = static_cast<QnTarget*>(t)->step(tok); if ((int)lg.size() != n) return -2; std::memcpy(logits, lg.data(), lg.size() * 4); return 0; } catch (const pyre_b200::Error& e) { return e.status; }
}
int shim_verify(void* t, const unsigned* toks, int nt, float* logits, int n) {
    try {
        auto rows = static_cast<QnTarget*>(t)->verify(std::vector<uint32_t>(toks, toks + nt));
        for (int j = 0; j < nt; j++) { if ((int)rows[j].size() != n) return -2; std::memcpy(logits + (size_t)j * n, rows[j].data(), (size_t)n * 4); }
        return 0;
    } catch (const pyre_b200::Error& e) { return e.status; }
}
int shim_keep(void* t, int nt, int keep) {
    try { static_cast<QnTarget*>(t)->keep(nt, keep); return 0; } catch (const pyre_b200::Error& e) { return e.status; }
}
// drafts with a sampler that always takes the row of the SECOND largest logit and reports a two-entry distribution; returns the number
// of drafts, -1 when no drafter is attached; q_sizes[j] = entries of draft j's distribution
int shim_draft(void* t, const unsigned* history, int nh, int k, float min_p, int sampled, unsigned* ids, int* q_sizes) {
    try {
        pyre_b200::DraftSampler second = [](const float* lg, const uint32_t* vid, int n) {
            int a = 0, b = -1;
            for (int i = 1; i < n; i++) { if (lg[i] > lg[a]) { b = a; a = i; } else if (b < 0 || lg[i] > lg[b]) b = i; }
            if (b < 0) b = a;
            return std::make_pair(vid[b], pyre_b200::Dist{{vid[a], 0.5f}, {vid[b], 0.5f}});
        };
        auto r = static_cast<QnTarget*>(t)->draft(std::vector<uint32_t>(history, history + nh), (size_t)k, min_p, sampled ? &second : nullptr);
        if (!r) return -1;
        for (size_t j = 0; j < r->size(); j++) { ids[j] = (*r)[j].token; q_sizes[j] = (*r)[j].q ? (int)(*r)[j].q->size() : 0; }
        return (int)r->size();
    } catch (const pyre_b200::Error& e) { return -100 - e.status; }
}
}
